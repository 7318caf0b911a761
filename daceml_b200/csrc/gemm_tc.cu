// fp16 GEMM on the 5th-generation tensor cores: C[M,N] = epilogue(alpha * A[M,K] . B), fp32 accumulate.
//
// One persistent CTA per SM, warp-specialised:
//   warp 0      TMA producer: streams 128x64 A tiles and BNx64 B tiles (128-byte swizzle) through a
//               ring of shared-memory stages, completion signalled on "full" mbarriers;
//   warp 1      owns the TMEM allocation and issues tcgen05.mma (128 x BN x 16) from one elected
//               thread; tcgen05.commit releases each stage ("empty") and publishes each finished
//               accumulator ("tmem_full");
//   warps 2-5   epilogue: tcgen05.ld the fp32 accumulator (one TMEM lane = one output row per
//               thread), apply alpha / bias / activation / residual, convert to fp16 and store.
// The accumulator is double-buffered in TMEM (2 x BN columns), so the epilogue of tile i overlaps
// the main loop of tile i+1.
//
// A is K-major ([M,K] row-major).  B is either K-major ([N,K] row-major, an nn.Linear weight or a
// Gemm with transB=1) or MN-major ([K,N] row-major, the ONNX MatMul operand); both are fed to the
// MMA directly, so no Transpose node has to run.  Two batch loops are folded into the TMA
// coordinates, which lets attention read Q, K, V per head straight out of a packed [T, 3H] buffer.
#include "gemm_common.cuh"

#include <stdlib.h>

namespace b200ml {

using namespace gemm;

namespace {

template <int BN>
struct GemmSmem {
    static constexpr int B_TILE_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
    static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
    static constexpr int OUT_BYTES = BN >= 128 ? EPI_WARPS * 32 * 128 : 0;  // a 32-row x 128-byte staging tile per epilogue warp
    static constexpr int BAR_BYTES = (2 * STAGES + 4) * 8 + 16;
    static constexpr int TOTAL = STAGES * STAGE_BYTES + OUT_BYTES + BAR_BYTES + 1024;  // + slack for 1024-byte alignment
};

// TMA_OUT: finished tiles leave through shared memory - each epilogue warp stages 32 rows x 64 columns
// (4 KB, in the 128-byte swizzle a tensor map expects) and one lane issues a bulk tensor store, instead
// of every lane writing 16-byte pieces of 32 different rows; ragged edges are clipped by the tensor map.
template <int BN, bool B_MN, bool TMA_OUT>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_f16_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const __grid_constant__ CUtensorMap tmap_c, const GemmArgs args) {
    static_assert(!TMA_OUT || BN >= 128, "the staged output path moves 64 columns per store");
    using S = GemmSmem<BN>;
    constexpr int STAGES = S::STAGES;
    constexpr uint32_t TMEM_COLS = 2 * BN;  // 128, 256 or 512: a power of two
    constexpr uint32_t IDESC = ptx::make_idesc_f16(BM, BN, 0, B_MN ? 1 : 0);

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
    const int num_kb = (args.k + BK - 1) / BK;

    if (warp == 0 && lane == 0) {
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
        if (TMA_OUT) ptx::prefetch_tensormap(&tmap_c);
    }
    if (warp == 1) {
        if (lane == 0) {
            for (int s = 0; s < STAGES; ++s) {
                ptx::mbar_init(&full_bar[s], 1);
                ptx::mbar_init(&empty_bar[s], 1);
            }
            for (int a = 0; a < 2; ++a) {
                ptx::mbar_init(&tmem_full_bar[a], 1);
                ptx::mbar_init(&tmem_empty_bar[a], EPI_WARPS);  // one arrival per epilogue warp
            }
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
    // A constant B (weights) does not depend on the kernel in front of this one: the B parts of the first tile's first
    // stages are requested before the dependency wait and stream in under the predecessor's tail (fresh stages: their
    // empty barriers pass); the A parts and everything else follow after the wait.
    const int early = (args.b_early && static_cast<int>(blockIdx.x) < args.num_tiles) ? (num_kb < STAGES ? num_kb : STAGES) : 0;
    if (warp == 0 && early > 0) {
        if (ptx::elect_one()) {
            const int rest = static_cast<int>(blockIdx.x) / args.tiles_m;
            const int nt = rest % args.tiles_n;
            const int batch = rest / args.tiles_n;
            const int bi = batch % args.batch_inner, bo = batch / args.batch_inner;
            const int n0 = nt * BN;
            for (int kb = 0; kb < early; ++kb) {
                uint8_t* sb = smem + kb * S::STAGE_BYTES + A_TILE_BYTES;
                ptx::mbar_expect_tx(&full_bar[kb], S::STAGE_BYTES);
                if (B_MN) {
#pragma unroll
                    for (int j = 0; j < BN / 64; ++j)
                        ptx::tma_load_4d(sb + j * (64 * BK * 2), &tmap_b, &full_bar[kb], n0 + j * 64, kb * BK,
                                         bi * args.b_use_inner, bo * args.b_use_outer);
                } else {
                    ptx::tma_load_4d(sb, &tmap_b, &full_bar[kb], kb * BK, n0, bi * args.b_use_inner, bo * args.b_use_outer);
                }
            }
        }
        __syncwarp();
    }
    pdl_wait();  // everything above overlaps the previous kernel's tail

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (ptx::elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            long long tr_wait = 0;
            const long long tr_begin = clock64();
            for (int tile = blockIdx.x; ok && tile < args.num_tiles; tile += gridDim.x) {
                const int mt = tile % args.tiles_m;
                const int rest = tile / args.tiles_m;
                const int nt = rest % args.tiles_n;
                const int batch = rest / args.tiles_n;
                const int bi = batch % args.batch_inner;
                const int bo = batch / args.batch_inner;
                const int m0 = mt * BM, n0 = nt * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    TRACE_T0();
                    if (!ptx::mbar_wait(&empty_bar[stage], phase ^ 1)) {
                        atomicExch(args.status, DEV_TIMEOUT_PRODUCER);
                        ok = false;
                        break;
                    }
                    TRACE_ADD(tr_wait);
                    uint8_t* sa = smem + stage * S::STAGE_BYTES;
                    uint8_t* sb = sa + A_TILE_BYTES;
                    const bool b_done = tile == static_cast<int>(blockIdx.x) && kb < early;  // requested before the dependency wait
                    if (!b_done) ptx::mbar_expect_tx(&full_bar[stage], S::STAGE_BYTES);
                    ptx::tma_load_4d(sa, &tmap_a, &full_bar[stage], kb * BK, m0, bi * args.a_use_inner,
                                     bo * args.a_use_outer);
                    if (b_done) {
                    } else if (B_MN) {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            ptx::tma_load_4d(sb + j * (64 * BK * 2), &tmap_b, &full_bar[stage], n0 + j * 64, kb * BK,
                                             bi * args.b_use_inner, bo * args.b_use_outer);
                    } else {
                        ptx::tma_load_4d(sb, &tmap_b, &full_bar[stage], kb * BK, n0, bi * args.b_use_inner,
                                         bo * args.b_use_outer);
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
#ifdef B200ML_TRACE
            args.trace[blockIdx.x * 16 + 0] = tr_wait;
            args.trace[blockIdx.x * 16 + 1] = clock64() - tr_begin;
#endif
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (ptx::elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            long long tr_wait_acc = 0, tr_wait_full = 0;
            const long long tr_begin = clock64();
            const unsigned long long tr_gt0 = ptx::global_timer_ns();
            for (int tile = blockIdx.x; ok && tile < args.num_tiles; tile += gridDim.x) {
                {
                    TRACE_T0();
                    if (!ptx::mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1)) {
                        atomicExch(args.status, DEV_TIMEOUT_MMA);
                        break;
                    }
                    TRACE_ADD(tr_wait_acc);
                }
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    {
                        TRACE_T0();
                        if (!ptx::mbar_wait(&full_bar[stage], phase)) {
                            atomicExch(args.status, DEV_TIMEOUT_MMA);
                            ok = false;
                            break;
                        }
                        TRACE_ADD(tr_wait_full);
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
                        ptx::mma_f16_ss(d_tmem, a_desc, b_desc, IDESC, (kb | kk) != 0 ? 1u : 0u);
                    }
                    ptx::mma_commit(&empty_bar[stage]);  // stage reusable once these MMAs have read it
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                ptx::mma_commit(&tmem_full_bar[acc]);
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1;
            }
#ifdef B200ML_TRACE
            args.trace[blockIdx.x * 16 + 2] = tr_wait_acc;
            args.trace[blockIdx.x * 16 + 3] = tr_wait_full;
            args.trace[blockIdx.x * 16 + 4] = clock64() - tr_begin;
            args.trace[blockIdx.x * 16 + 8] = (long long)(ptx::global_timer_ns() - tr_gt0);
#endif
        }
    } else {
        // ------------------------------ epilogue ------------------------------
        const int quarter = warp & 3;         // the TMEM lane quarter this warp may read
        const int half = (warp - 2) >> 2;     // which half of the tile's columns this warp finishes
        constexpr int WCOLS = BN / 2;         // columns per warp
        constexpr int CHUNKS = WCOLS / 32;    // 32-column chunks per warp: 1, 2 or 4
        constexpr int GROUP = CHUNKS >= 2 ? 2 : 1;  // chunks fetched per tcgen05.wait::ld
        const int row_in_tile = quarter * 32 + lane;
        int acc = 0;
        uint32_t acc_phase = 0;
        EpilogueParams ep;
        ep.flags = args.epilogue;
        ep.alpha = args.alpha;
        ep.bias_scale = args.bias_scale;
        ep.residual_scale = args.residual_scale;
        long long tr_wait_epi = 0, tr_ld = 0;
        const long long tr_begin = clock64();
        (void)tr_wait_epi, (void)tr_ld, (void)tr_begin;
        for (int tile = blockIdx.x; tile < args.num_tiles; tile += gridDim.x) {
            const int mt = tile % args.tiles_m;
            const int rest = tile / args.tiles_m;
            const int nt = rest % args.tiles_n;
            const int batch = rest / args.tiles_n;
            const int bi = batch % args.batch_inner;
            const int bo = batch / args.batch_inner;
            const int row = mt * BM + row_in_tile;
            const int n0 = nt * BN + half * WCOLS;
            {
                TRACE_T0();
                if (!ptx::mbar_wait(&tmem_full_bar[acc], acc_phase)) {
                    if (lane == 0) atomicExch(args.status, DEV_TIMEOUT_EPILOGUE);
                    break;
                }
                TRACE_ADD(tr_wait_epi);
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
                        ptx::tma_store_4d(&tmap_c, out_stage + (warp - 2) * 4096, col0, mt * BM + quarter * 32, bi, bo);
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
                {
                    TRACE_T0();
#pragma unroll
                    for (int u = 0; u < GROUP; ++u) ptx::tmem_ld_32x32b_x32(t_base + (c + u) * 32, r[u]);
                    if (row_ok) {
#pragma unroll
                        for (int u = 0; u < GROUP; ++u)
                            epilogue_prefetch_32(ep, pf[u], r_row, args.bias, col0 + u * 32, args.n, vec);
                    }
                    ptx::tmem_ld_wait();
                    TRACE_ADD(tr_ld);
                }
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
            if (lane == 0) ptx::mbar_arrive(&tmem_empty_bar[acc]);
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1;
        }
        if (TMA_OUT && lane == 0) ptx::tma_store_wait<0>();  // every bulk store of this warp has landed
#ifdef B200ML_TRACE
        if (threadIdx.x == 64) {
            args.trace[blockIdx.x * 16 + 5] = tr_wait_epi;
            args.trace[blockIdx.x * 16 + 6] = tr_ld;
            args.trace[blockIdx.x * 16 + 7] = clock64() - tr_begin;
        }
#endif
    }

    // ------------------------------ teardown ------------------------------
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        if (*reinterpret_cast<volatile int32_t*>(args.status) != DEV_OK) {
            // A wait gave up: give copies and MMAs still in flight time to land before the
            // tensor memory and shared memory are released.
            for (int i = 0; i < 200; ++i) __nanosleep(1000);
        }
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <int BN, bool B_MN, bool TMA_OUT>
int launch_impl(const b200ml_ctx* ctx, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, GemmArgs& args,
                cudaStream_t stream) {
    using S = GemmSmem<BN>;
    auto kernel = gemm_f16_tc_kernel<BN, B_MN, TMA_OUT>;
    static bool configured[64] = {};  // per instantiation and device
    if (!configured[ctx->device & 63]) {
        B200ML_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
        configured[ctx->device & 63] = true;
    }
    const int grid = args.num_tiles < ctx->sm_count ? args.num_tiles : ctx->sm_count;
    B200ML_CUDA(launch_pdl(kernel, dim3(grid), dim3(GEMM_THREADS), S::TOTAL, stream, ta, tb, tc, args));
    return check_launch("gemm_f16_tc");
}

template <int BN, bool B_MN>
int launch(const b200ml_ctx* ctx, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, GemmArgs& args,
           cudaStream_t stream) {
    if constexpr (BN >= 128) {
        if (args.tma_store) return launch_impl<BN, B_MN, true>(ctx, ta, tb, tc, args, stream);
    }
    return launch_impl<BN, B_MN, false>(ctx, ta, tb, tc, args, stream);
}

}  // namespace

int gemm_f16_simt(const b200ml_ctx* ctx, const b200ml_gemm_params* p, cudaStream_t stream);
int gemm_f16_pair(const b200ml_ctx* ctx, const b200ml_gemm_params* p, GemmArgs& args, int bn, cudaStream_t stream);

// B200ML_GEMM_PAIR=0 keeps every GEMM on the one-CTA kernel (for A/B comparisons).
static int pair_mode() {
    static const int mode = [] {
        const char* e = getenv("B200ML_GEMM_PAIR");
        return e ? atoi(e) : 1;
    }();
    return mode;
}
static bool pair_enabled() { return pair_mode() != 0; }

// Tile width.  The main loop of a 128 x 256 tile needs 48 KB per 64-deep k-block, which is what one
// SM can pull from L2 in the time the tensor core takes; narrower tiles are load-bound, so they
// are used only for narrow outputs.
static int pick_bn(int64_t n) { return n > 128 ? 256 : (n > 64 ? 128 : 64); }

int gemm_f16(const b200ml_ctx* ctx, const b200ml_gemm_params* p, cudaStream_t stream) {
    const int64_t batches = p->batch_outer * p->batch_inner;
    // Operand layouts the tensor-core kernel cannot address go to the FP32-FMA kernel instead.
    const bool a_ok = p->a_layout == 0 && aligned16(p->a) && p->lda % 8 == 0 && p->a_stride_inner % 8 == 0 &&
                      p->a_stride_outer % 8 == 0;
    const bool b_ok = aligned16(p->b) && p->ldb % 8 == 0 && p->b_stride_inner % 8 == 0 && p->b_stride_outer % 8 == 0;
    if (!a_ok || !b_ok || p->m * p->n * batches < 64 * 64) return gemm_f16_simt(ctx, p, stream);

    const int bn = pick_bn(p->n);
    GemmArgs args{};
    args.m = (int32_t)p->m;
    args.n = (int32_t)p->n;
    args.k = (int32_t)p->k;
    args.tiles_m = (int32_t)ceil_div(p->m, BM);
    args.tiles_n = (int32_t)ceil_div(p->n, bn);
    const int64_t tiles = (int64_t)args.tiles_m * args.tiles_n * batches;
    B200ML_REQUIRE(tiles < (1ll << 31), "gemm f16: too many tiles");
    args.num_tiles = (int32_t)tiles;
    args.batch_inner = (int32_t)p->batch_inner;
    args.epilogue = p->epilogue;
    args.a_use_inner = (p->batch_inner > 1 && p->a_stride_inner != 0) ? 1 : 0;
    args.a_use_outer = (p->batch_outer > 1 && p->a_stride_outer != 0) ? 1 : 0;
    args.b_use_inner = (p->batch_inner > 1 && p->b_stride_inner != 0) ? 1 : 0;
    args.b_use_outer = (p->batch_outer > 1 && p->b_stride_outer != 0) ? 1 : 0;
    args.ldc = p->ldc;
    args.c_so = p->c_stride_outer;
    args.c_si = p->c_stride_inner;
    args.ldr = p->ldr;
    args.r_so = p->r_stride_outer;
    args.r_si = p->r_stride_inner;
    args.alpha = p->alpha;
    args.bias_scale = p->bias_scale;
    args.residual_scale = p->residual_scale;
    args.c = static_cast<__half*>(p->c);
    args.bias = static_cast<const __half*>(p->bias);
    args.residual = static_cast<const __half*>(p->residual);
    args.status = ctx->status_dev;
    args.b_early = (p->flags & B200ML_GEMM_B_CONSTANT) ? 1 : 0;
#ifdef B200ML_TRACE
    args.trace = static_cast<long long*>(ctx->workspace);  // instrumented builds only: per-CTA cycle counters
#else
    args.trace = nullptr;
#endif
    bool vec = aligned16(p->c) && p->ldc % 8 == 0 && p->c_stride_inner % 8 == 0 && p->c_stride_outer % 8 == 0;
    if (p->residual)
        vec = vec && aligned16(p->residual) && p->ldr % 8 == 0 && p->r_stride_inner % 8 == 0 && p->r_stride_outer % 8 == 0;
    if (p->bias) vec = vec && aligned16(p->bias);
    args.vec_ok = vec ? 1 : 0;

    // Outputs with more 256-row tiles than CTA pairs go to the pair kernel (a third less operand
    // traffic per SM, and the epilogue of one tile overlaps the main loop of the next).  With at most
    // one tile per pair nothing overlaps and the one-CTA kernel, which spreads the same work over
    // twice as many independent tiles, is faster.
    const int64_t pair_tiles = ceil_div(p->m, 2 * BM) * args.tiles_n * batches;
    if (pair_enabled() && p->m > BM && bn >= 128 && (pair_tiles > ctx->sm_count / 2 || pair_mode() == 2)) {
        args.tiles_m = (int32_t)ceil_div(p->m, 2 * BM);
        args.num_tiles = (int32_t)pair_tiles;
        return gemm_f16_pair(ctx, p, args, bn, stream);
    }

    CUtensorMap ta, tb, tc;
    int rc = make_tmap(ctx, &ta, p->a, p->k, p->m, p->lda, p->batch_inner, p->a_stride_inner, p->batch_outer,
                       p->a_stride_outer, BK, BM, "A");
    if (rc) return rc;
    // C leaves through bulk tensor stores (64 columns x 32 rows per store) when its rows are 16-byte aligned
    // and N is a whole number of 64-column pieces; otherwise the warps store their rows themselves.
    args.tma_store = 0;
    tc = ta;
    if (bn >= 128 && args.vec_ok && p->n % 64 == 0) {
        rc = make_tmap(ctx, &tc, p->c, p->n, p->m, p->ldc, p->batch_inner, p->c_stride_inner, p->batch_outer,
                       p->c_stride_outer, 64, 32, "C");
        if (rc) return rc;
        args.tma_store = 1;
    }
    if (p->b_layout == 1) {
        rc = make_tmap(ctx, &tb, p->b, p->k, p->n, p->ldb, p->batch_inner, p->b_stride_inner, p->batch_outer,
                       p->b_stride_outer, BK, bn, "B");
        if (rc) return rc;
        switch (bn) {
            case 256: return launch<256, false>(ctx, ta, tb, tc, args, stream);
            case 128: return launch<128, false>(ctx, ta, tb, tc, args, stream);
            default: return launch<64, false>(ctx, ta, tb, tc, args, stream);
        }
    } else {
        rc = make_tmap(ctx, &tb, p->b, p->n, p->k, p->ldb, p->batch_inner, p->b_stride_inner, p->batch_outer,
                       p->b_stride_outer, 64, BK, "B");
        if (rc) return rc;
        switch (bn) {
            case 256: return launch<256, true>(ctx, ta, tb, tc, args, stream);
            case 128: return launch<128, true>(ctx, ta, tb, tc, args, stream);
            default: return launch<64, true>(ctx, ta, tb, tc, args, stream);
        }
    }
}

}  // namespace b200ml
