// 1x1 stride-1 convolution (NCHW, fp32) on the tensor cores with fp32-grade accuracy ("3 x TF32"):
//     Y[n, m, p] = act(B[m] + sum_c W[m, c] * gate[n, c] * X[n, c, p]) + R[n, m, p],    p = pixel of the H x W plane
// (the reference's route for this operator is cuDNN, daceml/onnx/op_implementations/cudnn_implementations.py:123-410;
// its pure route the loop nest of img_op_implementations.py:217-288).
//
// Per image this is the matrix product  D[pixel, m] = X[n]^T[pixel, c] . W^T[c, m]  with
//   * the 128 pixels of a tile as the M dimension (one TMEM lane per pixel),
//   * the output channels as N (one TMEM column each),
//   * the input channels as K, plus one more K row of ones against the bias (the bias add costs no instruction).
// X stays in NCHW: a TMA box {32 pixels, 32 channels} of the [N][C][HW] tensor lands in shared memory as 32 rows (one
// per channel) of 128 bytes (32 consecutive pixels) in the 128-byte swizzle with 32-byte atoms, which is the MN-major
// operand layout tcgen05.mma takes for 32-bit types (atoms of 4 K-rows x 128 bytes; four boxes make the 128-pixel tile).
// No layout change, no im2col: X is read once, Y written once.
//
// A single TF32 product keeps 11 bits of each operand (relative error ~5e-4), outside the 1e-4 the fp32 configurations
// allow, so each operand is split into hi (its leading TF32 bits) and lo = value - hi (exact), and the tensor core
// accumulates X_lo.W_hi + X_hi.W_lo + X_hi.W_hi in fp32 TMEM (the dropped lo.lo term is below 1e-6 of the operands'
// product).  The weights and the bias are split once per call by a small kernel (a few KB); X is split inside this
// kernel: two groups of four warps, taking the pipeline stages in turn, read the tile the TMA delivered, apply the
// squeeze-excite gate, write hi over it and lo next to it, and hand the stage to the MMA warp.
//
// Roles (832 threads, one persistent CTA per SM, tiles dealt round-robin): warp 0 TMA producer, warp 1 MMA issuer and
// TMEM owner, warps 2-9 split, warps 10-25 epilogue.  Split and epilogue are element-wise work whose chain of dependent
// instructions per value is long; they get their throughput from many warps and from straight-line code (activation
// and residual are template arguments of the inner loops).  Two accumulators in TMEM: tile i's epilogue runs under
// tile i+1's loads and products.  An epilogue warp owns 32 pixels (its TMEM lane quarter) and every fourth 8-channel
// unit: it reads two units (tcgen05.ld 32x32b.x8), applies activation and residual, writes them to its own 2 KB of
// shared memory as two [8 channels][32 pixels] boxes, and one lane sends them to Y with two bulk tensor stores, which
// also clip pixels past the plane and channels past M.  No per-value address arithmetic, no per-value predicate.
// The kernel is bound by HBM (X once, Y once).
#include "conv_tc.cuh"

namespace b200ml {

using namespace convtc;

namespace {

constexpr int PW_KB = 32;                            // channels per k-block: 32 fp32 = one 128-byte swizzle row of W
constexpr int PW_UMMA_K = 8;                         // tf32: 8 elements per instruction
constexpr int PW_STAGES = 4;
constexpr int PW_BOX_BYTES = 32 * PW_KB * 4;         // 4 KB: 32 pixels x 32 channels
constexpr int PW_TILE_BYTES = PW_BM * PW_KB * 4;     // 16 KB: X as delivered, overwritten by its hi part
constexpr int PW_STAGE_BYTES = 2 * PW_TILE_BYTES;    // ... and the lo part next to it
constexpr int PW_SPLIT_WARPS = 8, PW_SPLIT_GROUPS = 2, PW_EPI_WARPS = 16;
constexpr int PW_FIRST_EPI = 2 + PW_SPLIT_WARPS;
constexpr int PW_THREADS = 32 * (2 + PW_SPLIT_WARPS + PW_EPI_WARPS);
constexpr int PW_MAX_WEIGHT_BYTES = 64 * 1024;       // hi + lo of the padded weight matrix, resident in shared memory
constexpr int PW_OUT_BYTES = 2 * 8 * 32 * 4;         // per epilogue warp: two [8 channels][32 pixels] boxes
constexpr int PW_BAR_BYTES = 256;

struct PwArgs {
    int32_t c, m, hw, pblocks, num_tiles, kblocks, npad, act;
    const float* gate;      // [N, C] or null
    const float* residual;  // like Y or null
    int32_t* status;
};

// W [m, c], B [m] -> out [2][npad][kpad]: hi and lo parts, the bias as column c (it meets the row of ones the main
// kernel appends to X), zero-padded to whole 16-row / 32-column blocks.  Rounded to nearest here (|lo| <= 2^-11 |w|).
__global__ void __launch_bounds__(256) pw_split_weights_kernel(const float* __restrict__ w, const float* __restrict__ bias,
                                                               float* __restrict__ out, int m, int c, int npad, int kpad) {
    const int total = npad * kpad;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int row = i / kpad, k = i - row * kpad;
        float v = 0.0f;
        if (row < m) v = k < c ? __ldg(w + static_cast<int64_t>(row) * c + k) : ((k == c && bias) ? __ldg(bias + row) : 0.0f);
        const uint32_t b = __float_as_uint(v);
        const bool finite = (b & 0x7f800000u) != 0x7f800000u;
        const float hi = __uint_as_float(finite ? ((b + 0xfffu + ((b >> 13) & 1u)) & 0xffffe000u) : b);
        out[i] = hi;
        out[total + i] = finite ? v - hi : 0.0f;
    }
}

__global__ void __launch_bounds__(PW_THREADS, 1)
conv1x1_tf32x3_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                      const __grid_constant__ CUtensorMap tmap_y, const PwArgs args) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int w_part_bytes = args.npad * 128;                         // one k-block of W_hi (or W_lo): npad rows of 128 bytes
    uint8_t* out_stage = smem + PW_STAGES * PW_STAGE_BYTES;           // [epilogue warp][2][8][32]
    uint8_t* wsm = out_stage + PW_EPI_WARPS * PW_OUT_BYTES;           // [kblocks][2][npad][32]
    uint64_t* raw_full = reinterpret_cast<uint64_t*>(wsm + args.kblocks * 2 * w_part_bytes);
    uint64_t* ready = raw_full + PW_STAGES;
    uint64_t* empty = ready + PW_STAGES;
    uint64_t* w_full = empty + PW_STAGES;
    uint64_t* tmem_full = w_full + 1;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    uint32_t tmem_cols = 32;
    while (tmem_cols < 2u * args.npad) tmem_cols <<= 1;
    const uint32_t acc_stride = tmem_cols / 2;  // the two accumulators start on power-of-two columns
    const int kb_ones = args.c / PW_KB, row_ones = args.c % PW_KB;  // where the row of ones (against the bias) sits

    if (warp == 0 && lane == 0) {
        ptx::prefetch_tensormap(&tmap_x);
        ptx::prefetch_tensormap(&tmap_w);
        ptx::prefetch_tensormap(&tmap_y);
    }
    if (warp == 1) {
        if (lane == 0) {
            for (int s = 0; s < PW_STAGES; ++s) {
                ptx::mbar_init(&raw_full[s], 1);
                ptx::mbar_init(&ready[s], PW_SPLIT_WARPS / PW_SPLIT_GROUPS);
                ptx::mbar_init(&empty[s], 1);
            }
            ptx::mbar_init(w_full, 1);
            for (int a = 0; a < 2; ++a) {
                ptx::mbar_init(&tmem_full[a], 1);
                ptx::mbar_init(&tmem_empty[a], PW_EPI_WARPS);
            }
            ptx::fence_mbar_init();
        }
        __syncwarp();
        ptx::tmem_alloc(tmem_slot, tmem_cols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();  // the split weights (and possibly X, the gate, the residual) come from kernels before this one in the stream

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (ptx::elect_one()) {
            ptx::mbar_expect_tx(w_full, static_cast<uint32_t>(args.kblocks * 2 * w_part_bytes));
            for (int kb = 0; kb < args.kblocks; ++kb)
                for (int part = 0; part < 2; ++part)
                    ptx::tma_load_4d(wsm + (kb * 2 + part) * w_part_bytes, &tmap_w, w_full, kb * PW_KB, 0, part, 0);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < args.num_tiles; tile += gridDim.x) {
                const int n = tile / args.pblocks, p0 = (tile - n * args.pblocks) * PW_BM;
                for (int kb = 0; kb < args.kblocks; ++kb) {
                    if (!ptx::mbar_wait_suspend(&empty[stage], phase ^ 1)) {
                        atomicExch(args.status, DEV_TIMEOUT_PRODUCER);
                        ok = false;
                        break;
                    }
                    uint8_t* s0 = smem + stage * PW_STAGE_BYTES;
                    ptx::mbar_expect_tx(&raw_full[stage], PW_TILE_BYTES);
#pragma unroll
                    for (int j = 0; j < PW_BM / 32; ++j)  // pixels past the plane and channels past C arrive as zeros
                        ptx::tma_load_4d(s0 + j * PW_BOX_BYTES, &tmap_x, &raw_full[stage], p0 + 32 * j, kb * PW_KB, n, 0);
                    if (++stage == PW_STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (ptx::elect_one()) {
            const uint32_t idesc = pw_idesc(static_cast<uint32_t>(args.npad));
            int stage = 0;
            uint32_t phase = 0;
            bool ok = ptx::mbar_wait(w_full, 0);
            if (!ok) atomicExch(args.status, DEV_TIMEOUT_MMA);
            int it = 0;
            for (int tile = blockIdx.x; ok && tile < args.num_tiles; tile += gridDim.x, ++it) {
                const int acc = it & 1;
                if (!ptx::mbar_wait_suspend(&tmem_empty[acc], ((it >> 1) & 1) ^ 1)) {
                    atomicExch(args.status, DEV_TIMEOUT_MMA);
                    break;
                }
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * acc_stride;
                for (int kb = 0; kb < args.kblocks; ++kb) {
                    if (!ptx::mbar_wait(&ready[stage], phase)) {
                        atomicExch(args.status, DEV_TIMEOUT_MMA);
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint32_t xh = ptx::smem_u32(smem + stage * PW_STAGE_BYTES), xl = xh + PW_TILE_BYTES;
                    const uint32_t wh = ptx::smem_u32(wsm + (kb * 2) * w_part_bytes), wl = wh + w_part_bytes;
                    const int left = args.c + 1 - kb * PW_KB;                       // K rows in use: the channels and the row of ones
                    const int steps = left >= PW_KB ? PW_KB / PW_UMMA_K : (left + PW_UMMA_K - 1) / PW_UMMA_K;
                    for (int kk = 0; kk < steps; ++kk) {
                        // X: MN-major, 32-pixel atoms PW_BOX_BYTES apart, 4-channel groups 512 bytes apart; 8 channels per step
                        const uint64_t d_xh = make_smem_desc_sw128_base32(xh + kk * 1024, PW_BOX_BYTES, 512);
                        const uint64_t d_xl = make_smem_desc_sw128_base32(xl + kk * 1024, PW_BOX_BYTES, 512);
                        // W: K-major, 8 channels = 32 bytes along the swizzle row
                        const uint64_t d_wh = ptx::make_smem_desc_sw128(wh + kk * (PW_UMMA_K * 4), 16, 1024);
                        const uint64_t d_wl = ptx::make_smem_desc_sw128(wl + kk * (PW_UMMA_K * 4), 16, 1024);
                        pw_mma(d_tmem, d_xl, d_wh, idesc, (kb | kk) != 0 ? 1u : 0u);  // the two small terms first
                        pw_mma(d_tmem, d_xh, d_wl, idesc, 1u);
                        pw_mma(d_tmem, d_xh, d_wh, idesc, 1u);
                    }
                    ptx::mma_commit(&empty[stage]);
                    if (++stage == PW_STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                ptx::mma_commit(&tmem_full[acc]);
            }
        }
    } else if (warp < PW_FIRST_EPI) {
        // ------------------------------ split: raw X -> hi (in place) and lo ------------------------------
        // Two groups of four warps take the stages in turn (even stages group 0, odd stages group 1), so that the load ->
        // arithmetic -> store latency of one stage passes under the work on the next.
        constexpr int NT = 32 * PW_SPLIT_WARPS / PW_SPLIT_GROUPS;  // threads per group
        constexpr int NPK = PW_TILE_BYTES / 16 / NT;               // 16-byte packets per thread and stage
        static_assert(PW_STAGES % PW_SPLIT_GROUPS == 0 && NT * 32 == PW_BOX_BYTES, "packet t + NT j: box j / 2, channel row t / 8 + 16 (j & 1)");
        const int group = (warp - 2) / (PW_SPLIT_WARPS / PW_SPLIT_GROUPS);
        const int t = threadIdx.x - 64 - group * NT;
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < args.num_tiles; tile += gridDim.x) {
            const int n = tile / args.pblocks;
            for (int kb = 0; kb < args.kblocks; ++kb) {
                if ((stage % PW_SPLIT_GROUPS) != group) {  // the other group's stage
                    if (++stage == PW_STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                    continue;
                }
                ok = __all_sync(0xffffffffu, ptx::mbar_wait_suspend(&raw_full[stage], phase));
                if (!ok) {
                    if (lane == 0) atomicExch(args.status, DEV_TIMEOUT_EPILOGUE);
                    break;
                }
                // explicit shared-memory accesses (a generic pointer would cost a generic load and its long latency class)
                const uint32_t hi = ptx::smem_u32(smem + stage * PW_STAGE_BYTES) + t * 16, lo = hi + PW_TILE_BYTES;
                // packet t + NT j sits at byte 16 t + 2048 j of the stage: box j / 2, channel row t / 8 (even j) or
                // t / 8 + 16 (odd j); the swizzle moves packets only inside a row
                const int row0 = t >> 3, row1 = row0 + 16;
                float g0 = 1.0f, g1 = 1.0f;
                if (args.gate) {
                    const int c0 = kb * PW_KB + row0, c1 = kb * PW_KB + row1;
                    g0 = c0 < args.c ? __ldg(args.gate + static_cast<int64_t>(n) * args.c + c0) : 0.0f;
                    g1 = c1 < args.c ? __ldg(args.gate + static_cast<int64_t>(n) * args.c + c1) : 0.0f;
                }
                // every packet is read before the first is written back: the reads are independent, while a read
                // placed after a write to the same buffer would have to wait for it
                float4 v[NPK];
#pragma unroll
                for (int j = 0; j < NPK; ++j) v[j] = ld_shared_v4(hi + j * (NT * 16));
#pragma unroll
                for (int j = 0; j < NPK; ++j) {
                    const float g = (j & 1) ? g1 : g0;
                    float4 h, l;
                    split_tf32(v[j].x * g, h.x, l.x);
                    split_tf32(v[j].y * g, h.y, l.y);
                    split_tf32(v[j].z * g, h.z, l.z);
                    split_tf32(v[j].w * g, h.w, l.w);
                    st_shared_v4(hi + j * (NT * 16), h);
                    st_shared_v4(lo + j * (NT * 16), l);
                }
                if (kb == kb_ones && (row0 == row_ones || row1 == row_ones)) {  // the row of ones that meets the bias column of W
                    const int odd = row1 == row_ones ? 1 : 0;
#pragma unroll
                    for (int j = 0; j < NPK; j += 2) {
                        st_shared_v4(hi + (j + odd) * (NT * 16), make_float4(1.0f, 1.0f, 1.0f, 1.0f));
                        st_shared_v4(lo + (j + odd) * (NT * 16), make_float4(0.0f, 0.0f, 0.0f, 0.0f));
                    }
                }
                ptx::fence_proxy_async_smem();  // the tensor core reads shared memory through the async proxy
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&ready[stage]);
                if (++stage == PW_STAGES) {
                    stage = 0;
                    phase ^= 1;
                }
            }
        }
    } else {
        // ------------------------------ epilogue: 32 pixels x every fourth 8-channel unit per warp ------------------------------
        const int quarter = warp & 3;                      // TMEM lanes [32 q, 32 q + 32): a warp may only touch its own quarter
        const int group = (warp - PW_FIRST_EPI) >> 2;      // units group, group + 4, ...
        constexpr int NGROUPS = PW_EPI_WARPS / 4;
        const int nunits = (args.m + 7) / 8;
        uint8_t* stg = out_stage + (warp - PW_FIRST_EPI) * PW_OUT_BYTES;
        const uint32_t stg_lane = ptx::smem_u32(stg) + lane * 4;
        int it = 0;
        for (int tile = blockIdx.x; tile < args.num_tiles; tile += gridDim.x, ++it) {
            const int acc = it & 1;
            const int n = tile / args.pblocks, p0 = (tile - n * args.pblocks) * PW_BM;
            if (!__all_sync(0xffffffffu, ptx::mbar_wait_suspend(&tmem_full[acc], (it >> 1) & 1))) {
                if (lane == 0) atomicExch(args.status, DEV_TIMEOUT_EPILOGUE);
                break;
            }
            ptx::tc_fence_after();
            const int px = p0 + quarter * 32;              // first pixel of this warp's 32
            const uint32_t t_base = tmem_base + acc * acc_stride + (static_cast<uint32_t>(quarter * 32) << 16);
            if (px < args.hw) {  // warp-uniform: a quarter wholly past the plane (last tile of an image) has nothing to store
                const bool p_ok = px + lane < args.hw;
                const float* res = args.residual ? args.residual + (static_cast<int64_t>(n) * args.m) * args.hw + px + lane : nullptr;
#pragma unroll 1
                for (int ua = group; ua < nunits; ua += 2 * NGROUPS) {
                    const int ub = ua + NGROUPS;
                    const bool two = ub < nunits;  // warp-uniform
                    const int ca = ua * 8, cb = two ? ub * 8 : ca;
                    uint32_t r[2][8];
                    float rv[2][8];
                    // the residual values first: independent loads whose latency passes once per turn
                    if (res) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            rv[0][j] = (p_ok && ca + j < args.m) ? __ldg(res + static_cast<int64_t>(ca + j) * args.hw) : 0.0f;
                            rv[1][j] = (p_ok && cb + j < args.m) ? __ldg(res + static_cast<int64_t>(cb + j) * args.hw) : 0.0f;
                        }
                    }
                    ptx::tmem_ld_32x32b_x8(t_base + ca, r[0]);
                    ptx::tmem_ld_32x32b_x8(t_base + cb, r[1]);
                    if (lane == 0) ptx::tma_store_wait_read<0>();  // the stores of the last turn have read the staging boxes
                    ptx::tmem_ld_wait();
                    __syncwarp();
                    if (res) {
                        if (args.act == B200ML_EPI_SWISH) pw_finish_turn<B200ML_EPI_SWISH, true>(r, rv, stg_lane);
                        else if (args.act == 0) pw_finish_turn<0, true>(r, rv, stg_lane);
                        else if (args.act == B200ML_EPI_RELU) pw_finish_turn<B200ML_EPI_RELU, true>(r, rv, stg_lane);
                        else pw_finish_turn<B200ML_EPI_GELU, true>(r, rv, stg_lane);
                    } else {
                        if (args.act == B200ML_EPI_SWISH) pw_finish_turn<B200ML_EPI_SWISH, false>(r, rv, stg_lane);
                        else if (args.act == 0) pw_finish_turn<0, false>(r, rv, stg_lane);
                        else if (args.act == B200ML_EPI_RELU) pw_finish_turn<B200ML_EPI_RELU, false>(r, rv, stg_lane);
                        else pw_finish_turn<B200ML_EPI_GELU, false>(r, rv, stg_lane);
                    }
                    ptx::fence_proxy_async_smem();  // the bulk stores read shared memory through the async proxy
                    __syncwarp();
                    if (lane == 0) {
                        ptx::tma_store_4d(&tmap_y, stg, px, ca, n, 0);               // pixels past HW and channels past M are clipped
                        if (two) ptx::tma_store_4d(&tmap_y, stg + 1024, px, cb, n, 0);
                        ptx::tma_store_commit();
                    }
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&tmem_empty[acc]);
        }
        if (lane == 0) ptx::tma_store_wait<0>();  // the bulk stores have landed before the CTA may leave
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        if (*reinterpret_cast<volatile int32_t*>(args.status) != DEV_OK) {
            for (int i = 0; i < 200; ++i) __nanosleep(1000);  // a wait gave up: let copies in flight land before the CTA leaves
        }
        ptx::tmem_dealloc(tmem_base, tmem_cols);
    }
}

bool conv_tc_enabled() {
    static const bool on = [] {
        const char* e = getenv("B200ML_CONV_TC");
        return !(e && e[0] == '0');
    }();
    return on;
}

int pw_smem_bytes(int64_t npad, int64_t kpad) {
    return (int)(PW_STAGES * PW_STAGE_BYTES + PW_EPI_WARPS * PW_OUT_BYTES + 2 * npad * kpad * 4 + PW_BAR_BYTES + 1024 /* alignment */);
}

}  // namespace

// Whether the tensor-core kernel covers this convolution (the caller uses the FP32-FMA kernels otherwise).
bool conv1x1_tensor_core_applies(const b200ml_ctx* ctx, const b200ml_conv_params* p) {
    if (!conv_tc_enabled() || p->dtype != B200ML_F32 || !ctx->encode_tiled) return false;
    if (p->kh != 1 || p->kw != 1 || p->group != 1) return false;
    if (p->stride_h != 1 || p->stride_w != 1 || p->dil_h != 1 || p->dil_w != 1) return false;
    if (p->pad_top || p->pad_left || p->pad_bottom || p->pad_right) return false;
    const int64_t hw = p->h * p->w;
    if (hw % 4 != 0 || !aligned16(p->x) || !aligned16(p->y)) return false;  // 16-byte strides and bases for the tensor maps
    if (p->c < 8 || p->m < 8 || p->m > 256) return false;                    // tiny reductions stay on the FP32 pipe
    const int64_t npad = ceil_div(p->m, 16) * 16, kpad = ceil_div(p->c + 1, PW_KB) * PW_KB;  // + 1: the row of ones for the bias
    if (2 * npad * kpad * 4 > PW_MAX_WEIGHT_BYTES) return false;             // the split weights must fit in shared memory
    if (2 * npad * kpad * 4 > ctx->workspace_bytes) return false;
    if (hw * p->n < 16 * 1024) return false;                                 // too little work for two launches
    if (hw >= (1ll << 31) || p->n * ceil_div(hw, PW_BM) >= (1ll << 31) || p->n * p->c >= (1ll << 31)) return false;
    if (p->n * p->c * hw * 4 >= (1ll << 40) || p->n * p->m * hw * 4 >= (1ll << 40)) return false;  // tensor-map strides are below 2^40 bytes
    return true;
}

// Bytes of the split weights (hi and lo of the padded [npad][kpad] matrix with the bias column).
int64_t conv1x1_pack_bytes(const b200ml_conv_params* p) {
    const int64_t npad = ceil_div(p->m, 16) * 16, kpad = ceil_div(p->c + 1, PW_KB) * PW_KB;
    return 2 * npad * kpad * 4;
}

int conv1x1_pack(const b200ml_ctx*, const b200ml_conv_params* p, void* dst, cudaStream_t stream) {
    const int npad = (int)(ceil_div(p->m, 16) * 16), kpad = (int)(ceil_div(p->c + 1, PW_KB) * PW_KB);
    pw_split_weights_kernel<<<(unsigned)ceil_div((int64_t)npad * kpad, 256), 256, 0, stream>>>(
        static_cast<const float*>(p->weight), static_cast<const float*>(p->bias), static_cast<float*>(dst), (int)p->m, (int)p->c, npad, kpad);
    return check_launch("pw_split_weights");
}

int conv1x1_tensor_core(const b200ml_ctx* ctx, const b200ml_conv_params* p, cudaStream_t stream) {
    const int64_t hw = p->h * p->w;
    const int npad = (int)(ceil_div(p->m, 16) * 16), kpad = (int)(ceil_div(p->c + 1, PW_KB) * PW_KB);
    float* wsplit = static_cast<float*>(ctx->workspace);
    if (p->packed_weight) {  // split once by the caller
        B200ML_REQUIRE(aligned16(p->packed_weight), "conv: the packed weights must be 16-byte aligned");
        wsplit = const_cast<float*>(static_cast<const float*>(p->packed_weight));
    } else {
        int rc = conv1x1_pack(ctx, p, wsplit, stream);
        if (rc) return rc;
    }

    CUtensorMap tx, tw, ty;
    {
        const cuuint64_t dims[4] = {(cuuint64_t)hw, (cuuint64_t)p->c, (cuuint64_t)p->n, 1};
        const cuuint64_t strides[3] = {(cuuint64_t)hw * 4, (cuuint64_t)hw * 4 * (cuuint64_t)p->c, (cuuint64_t)hw * 4 * (cuuint64_t)p->c * (cuuint64_t)p->n};
        const cuuint32_t box[4] = {32, PW_KB, 1, 1};
        CUresult r = encode_tiled_cached(ctx, &tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, p->x, dims, strides, box,
                                         CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
        if (r != CUDA_SUCCESS) return fail(B200ML_ERR_CUDA, "conv 1x1: cuTensorMapEncodeTiled(X) failed with CUresult %d", (int)r);
    }
    {
        const cuuint64_t dims[4] = {(cuuint64_t)kpad, (cuuint64_t)npad, 2, 1};
        const cuuint64_t strides[3] = {(cuuint64_t)kpad * 4, (cuuint64_t)kpad * 4 * npad, (cuuint64_t)kpad * 4 * npad * 2};
        const cuuint32_t box[4] = {PW_KB, (cuuint32_t)npad, 1, 1};
        CUresult r = encode_tiled_cached(ctx, &tw, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, wsplit, dims, strides, box);
        if (r != CUDA_SUCCESS) return fail(B200ML_ERR_CUDA, "conv 1x1: cuTensorMapEncodeTiled(W) failed with CUresult %d", (int)r);
    }
    {
        const cuuint64_t dims[4] = {(cuuint64_t)hw, (cuuint64_t)p->m, (cuuint64_t)p->n, 1};
        const cuuint64_t strides[3] = {(cuuint64_t)hw * 4, (cuuint64_t)hw * 4 * (cuuint64_t)p->m, (cuuint64_t)hw * 4 * (cuuint64_t)p->m * (cuuint64_t)p->n};
        const cuuint32_t box[4] = {32, 8, 1, 1};
        CUresult r = encode_tiled_cached(ctx, &ty, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, p->y, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (r != CUDA_SUCCESS) return fail(B200ML_ERR_CUDA, "conv 1x1: cuTensorMapEncodeTiled(Y) failed with CUresult %d", (int)r);
    }
    PwArgs a{};
    a.c = (int32_t)p->c;
    a.m = (int32_t)p->m;
    a.hw = (int32_t)hw;
    a.pblocks = (int32_t)ceil_div(hw, PW_BM);
    a.num_tiles = (int32_t)(p->n * a.pblocks);
    a.kblocks = kpad / PW_KB;
    a.npad = npad;
    a.act = p->act & (B200ML_EPI_RELU | B200ML_EPI_SWISH | B200ML_EPI_GELU);
    a.gate = static_cast<const float*>(p->gate);
    a.residual = static_cast<const float*>(p->residual);
    a.status = ctx->status_dev;
    const int smem = pw_smem_bytes(npad, kpad);
    static int configured[64] = {};
    if (configured[ctx->device & 63] < smem) {
        B200ML_CUDA(cudaFuncSetAttribute(conv1x1_tf32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured[ctx->device & 63] = smem;
    }
    const int grid = a.num_tiles < ctx->sm_count ? a.num_tiles : ctx->sm_count;
    B200ML_CUDA(launch_pdl(conv1x1_tf32x3_kernel, dim3(grid), dim3(PW_THREADS), (size_t)smem, stream, tx, tw, ty, a));
    return check_launch("conv1x1_tf32x3");
}

}  // namespace b200ml
