// fp32 GEMM on the tensor cores with fp32-grade accuracy ("3 x TF32"):
//     C = act(alpha * A.B^T + bias) + residual,   A [M, K], B [N, K] (the nn.Linear layout) or [K, N] (ONNX MatMul), all fp32.
// A single TF32 product keeps 11 significant bits of each operand (relative error ~5e-4, outside the 1e-4 the fp32
// configurations allow).  Each operand is therefore split once, by a small kernel, into hi = the value rounded to
// TF32 and lo = value - hi (exact in fp32), and the tensor core accumulates
//     A_hi.B_hi + A_lo.B_hi + A_hi.B_lo          (the dropped A_lo.B_lo term is ~2^-22 relative)
// in fp32 TMEM.  Because hi is exactly representable in TF32, the result does not depend on how the hardware narrows
// its operands.  The tensor core's accumulator add truncates, and that error grows with the number of accumulation
// steps; the k-blocks are therefore dealt round-robin to four accumulators (all 512 TMEM columns), which the
// epilogue adds with round-to-nearest: a quarter of the steps per accumulator.  Same structure as the fp16 kernel: TMA producer warp (four tiles per stage), one MMA-issuing
// thread (tcgen05.mma kind::tf32, 128 x 128 x 8 per instruction), two accumulators in TMEM, eight epilogue warps.
// The split copies live in the context's workspace; the caller falls back to the FP32-FMA kernel when they do not
// fit, when A is not K-major, or when the product is too small to be worth three kernels.
#include "gemm_common.cuh"

namespace b200ml {

using namespace gemm;

namespace {

constexpr int TBM = 128, TBN = 128, TBK = 32;        // 32 fp32 = one 128-byte swizzle row
constexpr int T_UMMA_K = 8;                          // tf32: 8 elements = 32 bytes per instruction
constexpr int T_TILE_BYTES = TBM * TBK * 4;          // 16 KB (A and B tiles have the same shape)
constexpr int T_STAGE_BYTES = 4 * T_TILE_BYTES;      // A_hi, A_lo, B_hi, B_lo
constexpr int T_STAGES = 3;
constexpr int T_SMEM = T_STAGES * T_STAGE_BYTES + 256 + 1024;
constexpr int T_NACC = 4;                           // partial accumulators per tile
constexpr uint32_t T_TMEM_COLS = T_NACC * TBN;     // 512: one tile at a time, no overlap of epilogue and main loop
constexpr int T_PART_LD = TBM + 4;                  // row stride of a parked partial tile (column-major, padded)

// Instruction descriptor for kind::tf32: D = f32 (bits [4,6) = 1), A and B formats = tf32 (2 in [7,10) and [10,13)),
// both operands K-major, N >> 3 in [17,23), M >> 4 in [24,29).
constexpr uint32_t T_IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((TBN >> 3) << 17) | ((TBM >> 4) << 24);

struct Tf32Args {
    int32_t m, n, k, tiles_m, tiles_n, num_tiles;
    int32_t epilogue;
    float alpha, bias_scale, residual_scale;
    int64_t ldc, ldr;
    int32_t vec_ok;  // C (and residual) rows allow 16-byte accesses
    int32_t b_mn;    // B is [K, N] (N contiguous, the ONNX MatMul layout): the MN-major operand form
    float* c;
    const float* bias;
    const float* residual;
    int32_t* status;
};

__device__ __forceinline__ void mma_tf32_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Shared-memory descriptor of an MN-major 32-bit operand: the 128-byte swizzle with 32-byte atoms (layout type 1, the
// only one tcgen05.mma takes for MN-major tf32); atoms are 128 bytes (32 elements along N) x 4 k-rows, `lbo` apart along
// N and `sbo` apart along K.
__device__ __forceinline__ uint64_t make_smem_desc_mn32(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= 1ull << 46;
    d |= 1ull << 61;
    return d;
}

// hi = x rounded to nearest-even at 10 mantissa bits (TF32), lo = x - hi; rows of `cols` elements, source rows `ld` apart.
// One launch splits both operands of a product: the first `a_blocks` blocks take A, the others B.
struct SplitOperand {
    const float* x;
    float* hi;
    float* lo;
    int64_t rows, cols, ld;
};

__global__ void __launch_bounds__(256) split_tf32_kernel(const SplitOperand oa, const SplitOperand ob, unsigned a_blocks) {
    const bool first = blockIdx.x < a_blocks;
    const SplitOperand& o = first ? oa : ob;
    const float* __restrict__ x = o.x;
    float* __restrict__ hi = o.hi;
    float* __restrict__ lo = o.lo;
    const int64_t ld = o.ld;
    const int64_t n4 = o.rows * (o.cols / 4);
    const int64_t per_row = o.cols / 4;
    const int64_t block = first ? blockIdx.x : blockIdx.x - a_blocks;
    const int64_t nblocks = first ? a_blocks : gridDim.x - a_blocks;
    for (int64_t i = block * blockDim.x + threadIdx.x; i < n4; i += nblocks * blockDim.x) {
        const int64_t r = i / per_row, c4 = i - r * per_row;
        const float4 v = __ldg(reinterpret_cast<const float4*>(x + r * ld) + c4);
        const float in[4] = {v.x, v.y, v.z, v.w};
        float h[4], l[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t b = __float_as_uint(in[j]);
            const bool finite = (b & 0x7f800000u) != 0x7f800000u;
            const uint32_t rb = finite ? ((b + 0xfffu + ((b >> 13) & 1u)) & 0xffffe000u) : b;
            h[j] = __uint_as_float(rb);
            l[j] = finite ? in[j] - h[j] : 0.0f;
        }
        reinterpret_cast<float4*>(hi)[i] = make_float4(h[0], h[1], h[2], h[3]);
        reinterpret_cast<float4*>(lo)[i] = make_float4(l[0], l[1], l[2], l[3]);
    }
}

// Finishes NC columns of one output row: alpha, bias, activation, residual, store (16-byte stores when the row allows).
template <int NC>
__device__ __forceinline__ void tf32_finish_chunk(const Tf32Args& args, const uint32_t (&r)[NC], bool row_ok, float* c_row, const float* r_row,
                                                  int col0, bool has_bias, bool has_res, int act) {
    const bool full = args.vec_ok && col0 + NC <= args.n;
    if (!row_ok) return;
#pragma unroll
    for (int g = 0; g < NC / 4; ++g) {
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = args.alpha * __uint_as_float(r[g * 4 + j]);
        if (full) {
            if (has_bias) {
                const float4 b = __ldg(reinterpret_cast<const float4*>(args.bias + col0 + g * 4));
                v[0] = fmaf(args.bias_scale, b.x, v[0]), v[1] = fmaf(args.bias_scale, b.y, v[1]);
                v[2] = fmaf(args.bias_scale, b.z, v[2]), v[3] = fmaf(args.bias_scale, b.w, v[3]);
            }
            if (act) {
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = apply_act(v[j], act);
            }
            if (has_res) {
                const float4 q = __ldg(reinterpret_cast<const float4*>(r_row + col0 + g * 4));
                v[0] = fmaf(args.residual_scale, q.x, v[0]), v[1] = fmaf(args.residual_scale, q.y, v[1]);
                v[2] = fmaf(args.residual_scale, q.z, v[2]), v[3] = fmaf(args.residual_scale, q.w, v[3]);
            }
            *reinterpret_cast<float4*>(c_row + col0 + g * 4) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int col = col0 + g * 4 + j;
                if (col < args.n) {
                    float o = v[j];
                    if (has_bias) o = fmaf(args.bias_scale, __ldg(args.bias + col), o);
                    if (act) o = apply_act(o, act);
                    if (has_res) o = fmaf(args.residual_scale, __ldg(r_row + col), o);
                    c_row[col] = o;
                }
            }
        }
    }
}

// SPLITK > 1: a cluster of SPLITK CTAs shares one output tile, each CTA takes a contiguous share of the k-blocks; the
// partial tiles are parked in shared memory and every CTA adds up and finishes its own share of the tile's columns,
// reading the peers' partial tiles through distributed shared memory.  For products with few output tiles (a tall A against
// a narrow B), where one CTA per tile would leave most SMs idle and each busy SM bound by what it can take in from L2.
template <int SPLITK>
__global__ void __cluster_dims__(SPLITK, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap tmap_ah, const __grid_constant__ CUtensorMap tmap_al,
                   const __grid_constant__ CUtensorMap tmap_bh, const __grid_constant__ CUtensorMap tmap_bl, const Tf32Args args) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + T_STAGES * T_STAGE_BYTES);
    uint64_t* empty_bar = full_bar + T_STAGES;
    uint64_t* tmem_full_bar = empty_bar + T_STAGES;
    uint64_t* tmem_empty_bar = tmem_full_bar + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int num_kb = (args.k + TBK - 1) / TBK;
    const uint32_t rank = SPLITK > 1 ? ptx::cluster_ctarank() : 0u;
    const int first_tile = blockIdx.x / SPLITK, tile_step = gridDim.x / SPLITK;  // a cluster = a tile at a time
    const int kb_per = (num_kb + SPLITK - 1) / SPLITK;
    const int kb_begin = static_cast<int>(rank) * kb_per;
    const int kb_end = kb_begin + kb_per < num_kb ? kb_begin + kb_per : num_kb;
    float* partial = reinterpret_cast<float*>(smem);  // SPLITK > 1: the pipeline stages are idle by the time it is written

    if (warp == 0 && lane == 0) {
        ptx::prefetch_tensormap(&tmap_ah);
        ptx::prefetch_tensormap(&tmap_al);
        ptx::prefetch_tensormap(&tmap_bh);
        ptx::prefetch_tensormap(&tmap_bl);
    }
    if (warp == 1) {
        if (lane == 0) {
            for (int s = 0; s < T_STAGES; ++s) {
                ptx::mbar_init(&full_bar[s], 1);
                ptx::mbar_init(&empty_bar[s], 1);
            }
            ptx::mbar_init(&tmem_full_bar[0], 1);
            ptx::mbar_init(&tmem_empty_bar[0], EPI_WARPS);
            ptx::fence_mbar_init();
        }
        __syncwarp();
        ptx::tmem_alloc(tmem_slot, T_TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (ptx::elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = first_tile; ok && tile < args.num_tiles; tile += tile_step) {
                const int m0 = (tile % args.tiles_m) * TBM, n0 = (tile / args.tiles_m) * TBN;
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!ptx::mbar_wait(&empty_bar[stage], phase ^ 1)) {
                        atomicExch(args.status, DEV_TIMEOUT_PRODUCER);
                        ok = false;
                        break;
                    }
                    uint8_t* s0 = smem + stage * T_STAGE_BYTES;
                    ptx::mbar_expect_tx(&full_bar[stage], T_STAGE_BYTES);
                    ptx::tma_load_4d(s0, &tmap_ah, &full_bar[stage], kb * TBK, m0, 0, 0);
                    ptx::tma_load_4d(s0 + T_TILE_BYTES, &tmap_al, &full_bar[stage], kb * TBK, m0, 0, 0);
                    if (args.b_mn) {
                        // four boxes of 32 columns x 32 k-rows each: 32 lines of 128 bytes, the MN-major atom layout
                        for (int j = 0; j < TBN / 32; ++j) {
                            ptx::tma_load_4d(s0 + 2 * T_TILE_BYTES + j * 4096, &tmap_bh, &full_bar[stage], n0 + 32 * j, kb * TBK, 0, 0);
                            ptx::tma_load_4d(s0 + 3 * T_TILE_BYTES + j * 4096, &tmap_bl, &full_bar[stage], n0 + 32 * j, kb * TBK, 0, 0);
                        }
                    } else {
                        ptx::tma_load_4d(s0 + 2 * T_TILE_BYTES, &tmap_bh, &full_bar[stage], kb * TBK, n0, 0, 0);
                        ptx::tma_load_4d(s0 + 3 * T_TILE_BYTES, &tmap_bl, &full_bar[stage], kb * TBK, n0, 0, 0);
                    }
                    if (++stage == T_STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (ptx::elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int tile = first_tile; ok && tile < args.num_tiles; tile += tile_step) {
                if (!ptx::mbar_wait(&tmem_empty_bar[0], acc_phase ^ 1)) {
                    atomicExch(args.status, DEV_TIMEOUT_MMA);
                    break;
                }
                ptx::tc_fence_after();
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    const int kbl = kb - kb_begin;
                    const uint32_t d_tmem = tmem_base + (kbl % T_NACC) * TBN;  // this CTA's i-th k-block adds into accumulator i mod 4
                    if (!ptx::mbar_wait(&full_bar[stage], phase)) {
                        atomicExch(args.status, DEV_TIMEOUT_MMA);
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint32_t ah = ptx::smem_u32(smem + stage * T_STAGE_BYTES);
                    const uint32_t al = ah + T_TILE_BYTES, bh = ah + 2 * T_TILE_BYTES, bl = ah + 3 * T_TILE_BYTES;
#pragma unroll
                    for (int kk = 0; kk < TBK / T_UMMA_K; ++kk) {
                        const uint32_t off = kk * (T_UMMA_K * 4);  // 32 bytes along K inside the 128-byte swizzle row
                        const uint64_t d_ah = ptx::make_smem_desc_sw128(ah + off, 16, 1024);
                        const uint64_t d_al = ptx::make_smem_desc_sw128(al + off, 16, 1024);
                        // B K-major: 32 bytes along the swizzle row per step; B MN-major: 8 k-rows (two 512-byte groups) per
                        // step, 32-column atoms one box (4 KB) apart
                        const uint64_t d_bh = args.b_mn ? make_smem_desc_mn32(bh + kk * 1024, 4096, 512) : ptx::make_smem_desc_sw128(bh + off, 16, 1024);
                        const uint64_t d_bl = args.b_mn ? make_smem_desc_mn32(bl + kk * 1024, 4096, 512) : ptx::make_smem_desc_sw128(bl + off, 16, 1024);
                        const uint32_t idesc = args.b_mn ? (T_IDESC | (1u << 16)) : T_IDESC;
                        // the two small terms first, the large one last
                        mma_tf32_ss(d_tmem, d_al, d_bh, idesc, (kbl >= T_NACC || kk != 0) ? 1u : 0u);
                        mma_tf32_ss(d_tmem, d_ah, d_bl, idesc, 1u);
                        mma_tf32_ss(d_tmem, d_ah, d_bh, idesc, 1u);
                    }
                    ptx::mma_commit(&empty_bar[stage]);
                    if (++stage == T_STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                ptx::mma_commit(&tmem_full_bar[0]);
                acc_phase ^= 1;
            }
        }
    } else {
        // ------------------------------ epilogue: 32 rows x 64 columns per warp ------------------------------
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        const int row_in_tile = quarter * 32 + lane;
        uint32_t acc_phase = 0;
        const int nacc = kb_end - kb_begin < T_NACC ? kb_end - kb_begin : T_NACC;  // accumulators that received a k-block
        const bool has_bias = (args.epilogue & B200ML_EPI_BIAS) && args.bias != nullptr;
        const bool has_res = (args.epilogue & B200ML_EPI_RESIDUAL) && args.residual != nullptr;
        const int act = args.epilogue & (B200ML_EPI_RELU | B200ML_EPI_GELU | B200ML_EPI_SWISH);
        for (int tile = first_tile; tile < args.num_tiles; tile += tile_step) {
            const int row = (tile % args.tiles_m) * TBM + row_in_tile;
            const int n0 = (tile / args.tiles_m) * TBN + half * 64;
            if (!ptx::mbar_wait(&tmem_full_bar[0], acc_phase)) {
                if (lane == 0) atomicExch(args.status, DEV_TIMEOUT_EPILOGUE);
                break;
            }
            ptx::tc_fence_after();
            const bool row_ok = row < args.m;
            float* c_row = args.c + static_cast<int64_t>(row) * args.ldc;
            const float* r_row = has_res ? args.residual + static_cast<int64_t>(row) * args.ldr : nullptr;
            const uint32_t t_base = tmem_base + half * 64 + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {
                const int col0 = n0 + c * 32;
                if (col0 >= args.n) break;  // warp-uniform
                uint32_t r[32];
                __syncwarp();  // the TMEM load is warp-collective: no lane may still be inside the guarded stores below
                ptx::tmem_ld_32x32b_x32(t_base + c * 32, r);  // every lane loads; only the stores are guarded
                ptx::tmem_ld_wait();
                if (nacc == 0) {  // SPLITK: a CTA past the end of K received nothing; its share is zero
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = 0u;
                }
                for (int a = 1; a < nacc; ++a) {  // warp-uniform trip count
                    uint32_t q[32];
                    ptx::tmem_ld_32x32b_x32(t_base + a * TBN + c * 32, q);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(q[j]));
                }
                if constexpr (SPLITK == 1) {
                    tf32_finish_chunk<32>(args, r, row_ok, c_row, r_row, col0, has_bias, has_res, act);
                } else {
                    // this CTA's share of K: park the partial sums column-major (a lane = a row: conflict-free) for the reduction
#pragma unroll
                    for (int j = 0; j < 32; ++j) partial[(half * 64 + c * 32 + j) * T_PART_LD + row_in_tile] = __uint_as_float(r[j]);
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&tmem_empty_bar[0]);
            acc_phase ^= 1;
        }
    }

    if constexpr (SPLITK > 1) {
        // every thread of the cluster: the partial tiles are parked
        ptx::cluster_sync_acq_rel();
        if (warp >= 2 && first_tile < args.num_tiles) {
            // every rank adds up and finishes its own 128 / SPLITK columns of the tile: a warp takes 32 rows (a lane = a row,
            // so the loads from a peer's shared memory are 128 contiguous bytes) and half of those columns
            constexpr int NC = TBN / SPLITK / 2;
            const int quarter = warp & 3, half = (warp - 2) >> 2, row_in_tile = quarter * 32 + lane;
            const int tile = first_tile;
            const int row = (tile % args.tiles_m) * TBM + row_in_tile;
            const int tc0 = static_cast<int>(rank) * (TBN / SPLITK) + half * NC;  // first column inside the tile
            const int col0 = (tile / args.tiles_m) * TBN + tc0;
            const bool has_bias = (args.epilogue & B200ML_EPI_BIAS) && args.bias != nullptr;
            const bool has_res = (args.epilogue & B200ML_EPI_RESIDUAL) && args.residual != nullptr;
            const int act = args.epilogue & (B200ML_EPI_RELU | B200ML_EPI_GELU | B200ML_EPI_SWISH);
            float* c_row = args.c + static_cast<int64_t>(row) * args.ldc;
            const float* r_row = has_res ? args.residual + static_cast<int64_t>(row) * args.ldr : nullptr;
            if (col0 < args.n) {  // warp-uniform
                uint32_t r[NC];
#pragma unroll
                for (int j = 0; j < NC; ++j) {
                    const float* slot = partial + (tc0 + j) * T_PART_LD + row_in_tile;
                    float v = 0.0f;
#pragma unroll
                    for (int q = 0; q < SPLITK; ++q) v += ptx::ld_shared_cluster_f32(slot, q);  // rank order: the same sum on every run
                    r[j] = __float_as_uint(v);
                }
                tf32_finish_chunk<NC>(args, r, row < args.m, c_row, r_row, col0, has_bias, has_res, act);
            }
        }
        ptx::cluster_sync_acq_rel();  // no CTA leaves while a peer may still read its partial tile
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        if (*reinterpret_cast<volatile int32_t*>(args.status) != DEV_OK) {
            for (int i = 0; i < 200; ++i) __nanosleep(1000);
        }
        ptx::tmem_dealloc(tmem_base, T_TMEM_COLS);
    }
}

// rank-2 fp32 tensor map {K, rows} (as rank 4 with two unit dimensions), box 32 x 128, 128-byte swizzle.
int make_tmap_f32(const b200ml_ctx* ctx, CUtensorMap* out, const float* base, int64_t k, int64_t rows, const char* what) {
    if (!ctx->encode_tiled) return fail(B200ML_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const uint64_t row_bytes = static_cast<uint64_t>(k) * 4;
    const uint64_t dummy = row_bytes * static_cast<uint64_t>(rows);
    cuuint64_t dims[4] = {(cuuint64_t)k, (cuuint64_t)rows, 1, 1};
    cuuint64_t strides[3] = {row_bytes, dummy, dummy};
    cuuint32_t box[4] = {TBK, TBM, 1, 1};
    CUresult r = encode_tiled_cached(ctx, out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, base, dims, strides, box);
    if (r != CUDA_SUCCESS) return fail(B200ML_ERR_CUDA, "cuTensorMapEncodeTiled(%s, fp32) failed with CUresult %d", what, (int)r);
    return B200ML_OK;
}

bool splitk_enabled() {
    static const bool on = [] {
        const char* e = getenv("B200ML_TF32_SPLITK");
        return !(e && e[0] == '0');
    }();
    return on;
}

bool tf32x3_enabled() {
    static const bool on = [] {
        const char* e = getenv("B200ML_TF32X3");
        return !(e && e[0] == '0');
    }();
    return on;
}

}  // namespace

// Whether the tensor-core path covers this fp32 product (the caller uses the FP32-FMA kernel otherwise).
bool gemm_f32_tensor_core_applies(const b200ml_ctx* ctx, const b200ml_gemm_params* p) {
    if (!tf32x3_enabled() || p->batch_outer * p->batch_inner != 1) return false;
    if (p->a_layout != 0) return false;                                            // A K-major; B [N, K] or [K, N]
    if (p->k % 4 != 0 || p->lda % 4 != 0 || p->ldb % 4 != 0) return false;         // 16-byte rows for the split and the TMA
    if (p->b_layout == 0 && p->n % 4 != 0) return false;
    if (!aligned16(p->a) || !aligned16(p->b)) return false;
    if (p->m < 256 || p->n < 32 || p->k < 64) return false;                        // three launches must pay for themselves
    if (p->m * p->n * p->k < (1ll << 26)) return false;
    if (p->m >= (1ll << 24) || p->n >= (1ll << 24)) return false;
    const int64_t need = 2 * (p->m + p->n) * p->k * 4;
    return need <= ctx->workspace_bytes;
}

int gemm_f32_tensor_core(const b200ml_ctx* ctx, const b200ml_gemm_params* p, cudaStream_t stream) {
    float* ws = static_cast<float*>(ctx->workspace);
    float* a_hi = ws;
    float* a_lo = a_hi + p->m * p->k;
    float* b_hi = a_lo + p->m * p->k;
    float* b_lo = b_hi + p->n * p->k;
    const auto blocks = [&](int64_t elems) {
        int64_t b = ceil_div(elems / 4, 256);
        const int64_t cap = static_cast<int64_t>(ctx->sm_count) * 16;
        return static_cast<unsigned>(b < 1 ? 1 : (b > cap ? cap : b));
    };
    const unsigned ba = blocks(p->m * p->k), bb = blocks(p->n * p->k);
    const bool b_mn = p->b_layout == 0;  // B [K, N]: its split copies keep that shape, rows of N
    const SplitOperand oa{static_cast<const float*>(p->a), a_hi, a_lo, p->m, p->k, p->lda};
    const SplitOperand ob{static_cast<const float*>(p->b), b_hi, b_lo, b_mn ? p->k : p->n, b_mn ? p->n : p->k, p->ldb};
    split_tf32_kernel<<<ba + bb, 256, 0, stream>>>(oa, ob, ba);
    int rc = check_launch("split_tf32");
    if (rc) return rc;

    CUtensorMap tah, tal, tbh, tbl;
    if ((rc = make_tmap_f32(ctx, &tah, a_hi, p->k, p->m, "A hi"))) return rc;
    if ((rc = make_tmap_f32(ctx, &tal, a_lo, p->k, p->m, "A lo"))) return rc;
    if (b_mn) {
        for (int part = 0; part < 2; ++part) {
            const cuuint64_t dims[4] = {(cuuint64_t)p->n, (cuuint64_t)p->k, 1, 1};
            const cuuint64_t strides[3] = {(cuuint64_t)p->n * 4, (cuuint64_t)p->n * 4 * (cuuint64_t)p->k, (cuuint64_t)p->n * 4 * (cuuint64_t)p->k};
            const cuuint32_t box[4] = {32, TBK, 1, 1};
            CUresult r = encode_tiled_cached(ctx, part ? &tbl : &tbh, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, part ? b_lo : b_hi, dims, strides, box,
                                             CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
            if (r != CUDA_SUCCESS) return fail(B200ML_ERR_CUDA, "cuTensorMapEncodeTiled(B [K, N], fp32) failed with CUresult %d", (int)r);
        }
    } else {
        if ((rc = make_tmap_f32(ctx, &tbh, b_hi, p->k, p->n, "B hi"))) return rc;
        if ((rc = make_tmap_f32(ctx, &tbl, b_lo, p->k, p->n, "B lo"))) return rc;
    }

    Tf32Args args{};
    args.m = (int32_t)p->m;
    args.n = (int32_t)p->n;
    args.k = (int32_t)p->k;
    args.tiles_m = (int32_t)ceil_div(p->m, TBM);
    args.tiles_n = (int32_t)ceil_div(p->n, TBN);
    args.num_tiles = args.tiles_m * args.tiles_n;
    args.epilogue = p->epilogue;
    args.alpha = p->alpha;
    args.bias_scale = p->bias_scale;
    args.residual_scale = p->residual_scale;
    args.ldc = p->ldc;
    args.ldr = p->ldr;
    bool vec = aligned16(p->c) && p->ldc % 4 == 0;
    if (p->residual) vec = vec && aligned16(p->residual) && p->ldr % 4 == 0;
    if (p->bias) vec = vec && aligned16(p->bias);
    args.vec_ok = vec ? 1 : 0;
    args.b_mn = b_mn ? 1 : 0;
    args.c = static_cast<float*>(p->c);
    args.bias = static_cast<const float*>(p->bias);
    args.residual = static_cast<const float*>(p->residual);
    args.status = ctx->status_dev;

    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        B200ML_CUDA(cudaFuncSetAttribute(gemm_tf32x3_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, T_SMEM));
        B200ML_CUDA(cudaFuncSetAttribute(gemm_tf32x3_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, T_SMEM));
        B200ML_CUDA(cudaFuncSetAttribute(gemm_tf32x3_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, T_SMEM));
        configured[ctx->device & 63] = true;
    }
    // few output tiles: split K over a cluster of 2 or 4 CTAs per tile (one tile per cluster, no persistence)
    const int num_kb = (int)ceil_div(p->k, TBK);
    int split = 1;
    if (splitk_enabled()) {
        if (args.num_tiles * 4 <= ctx->sm_count && num_kb >= 8) split = 4;
        else if (args.num_tiles * 2 <= ctx->sm_count && num_kb >= 4) split = 2;
    }
    if (split == 4) B200ML_CUDA(launch_pdl(gemm_tf32x3_kernel<4>, dim3(args.num_tiles * 4), dim3(GEMM_THREADS), T_SMEM, stream, tah, tal, tbh, tbl, args));
    else if (split == 2) B200ML_CUDA(launch_pdl(gemm_tf32x3_kernel<2>, dim3(args.num_tiles * 2), dim3(GEMM_THREADS), T_SMEM, stream, tah, tal, tbh, tbl, args));
    else {
        const int grid = args.num_tiles < ctx->sm_count ? args.num_tiles : ctx->sm_count;
        B200ML_CUDA(launch_pdl(gemm_tf32x3_kernel<1>, dim3(grid), dim3(GEMM_THREADS), T_SMEM, stream, tah, tal, tbh, tbl, args));
    }
    return check_launch("gemm_tf32x3");
}

}  // namespace b200ml
