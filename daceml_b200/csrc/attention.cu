// Fused attention for fp16 tensors with head_dim 64: O = softmax(scale * Q K^T + mask) V.
//
// One CTA per (batch, head, 128 query rows); two CTAs share an SM so that one CTA's softmax
// overlaps the other's tensor-core work.  Per 128-key tile:
//   warp 0   TMA loads of Q (once), K_j and V_j straight from the caller's strided tensors
//            (so Q/K/V may live inside a packed [T, 3H] projection output - no head split);
//   warp 1   tcgen05.mma S = Q K_j^T (128x128x64) into TMEM, later O_j = P_j V_j (128x64x128);
//            V is consumed MN-major exactly as TMA lays it down - no transpose;
//   warps 2-9  two threads per query row (64 keys each): read S from TMEM, online softmax in the log2 domain,
//            write P_j (fp16) into shared memory in the 128-byte-swizzled K-major layout the MMA
//            reads, then fold O_j into the fp32 running output held in registers.
// The scores never touch HBM: traffic is Q, K, V in and O out.
#include "common.cuh"
#include "ptx.cuh"
#include "epilogue.cuh"
#include <math.h>

namespace b200ml {

namespace {

constexpr int AT_THREADS = 320;  // TMA warp, MMA warp, eight softmax warps
constexpr int QT = 128;   // query rows per CTA
constexpr int KT = 128;   // keys per iteration
constexpr int HD = 64;    // head dimension
constexpr int TILE_BYTES = 128 * HD * 2;         // 16 KB: Q, K_j or V_j
constexpr int P_BYTES = QT * KT * 2;             // 32 KB: two 64-column swizzle atoms
constexpr int XCHG_FLOATS = 768;                 // row maxima (two parities) and row sums exchanged between half-warps
constexpr int KV_SLOTS = 3;                      // K_0, V_0, K_1, V_1, ... travel through a ring of three tiles
constexpr int AT_SMEM = (1 + KV_SLOTS) * TILE_BYTES + P_BYTES + 256 + XCHG_FLOATS * 4 + 1024;
constexpr uint32_t AT_TMEM_COLS = 256;           // S: columns [0,128), O_j: [128,192)

struct AttnArgs {
    int32_t heads, seq_q, seq_kv, q_tiles;
    int64_t o_stride_b, o_stride_h, o_stride_s;
    float scale_log2;  // scale * log2(e)
    __half* o;
    const __half* mask;  // [batch, seq_kv] additive, or null
    int32_t* status;
    long long* trace;
};

#ifdef B200ML_TRACE
#define AT_MARK(i) do { const long long _n = clock64(); tr[i] += _n - tr_last; tr_last = _n; } while (0)
#else
#define AT_MARK(i)
#endif

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(AT_THREADS, 2)
attention_f16_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const AttnArgs args) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sq = smem;
    uint8_t* skv = smem + TILE_BYTES;  // KV_SLOTS tiles
    uint8_t* sp = smem + (1 + KV_SLOTS) * TILE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sp + P_BYTES);
    uint64_t* q_full = bars + 0;
    uint64_t* kv_full = bars + 1;                // [KV_SLOTS]
    uint64_t* kv_empty = bars + 1 + KV_SLOTS;    // [KV_SLOTS]
    uint64_t* s_full = bars + 1 + 2 * KV_SLOTS;
    uint64_t* p_full = s_full + 1;
    uint64_t* o_full = s_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 3);
    float* xchg = reinterpret_cast<float*>(sp + P_BYTES + 256);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int qt = blockIdx.x % args.q_tiles;
    const int bh = blockIdx.x / args.q_tiles;
    const int head = bh % args.heads;
    const int batch = bh / args.heads;
    const int q0 = qt * QT;
    const int n_kv = (args.seq_kv + KT - 1) / KT;

    if (warp == 0 && lane == 0) {
        ptx::prefetch_tensormap(&tmap_q);
        ptx::prefetch_tensormap(&tmap_k);
        ptx::prefetch_tensormap(&tmap_v);
    }
    if (warp == 1) {
        if (lane == 0) {
            ptx::mbar_init(q_full, 1);
            for (int i = 0; i < KV_SLOTS; ++i) {
                ptx::mbar_init(&kv_full[i], 1);
                ptx::mbar_init(&kv_empty[i], 1);
            }
            ptx::mbar_init(s_full, 1);
            ptx::mbar_init(p_full, 8);  // one arrival per softmax warp
            ptx::mbar_init(o_full, 1);
            ptx::fence_mbar_init();
        }
        __syncwarp();
        ptx::tmem_alloc(tmem_slot, AT_TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base;
    const uint32_t tmem_o = tmem_base + 128;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (ptx::elect_one()) {
            ptx::mbar_expect_tx(q_full, TILE_BYTES);
            ptx::tma_load_4d(sq, &tmap_q, q_full, 0, q0, head, batch);
            // item 2j is K_j, item 2j + 1 is V_j; item i lives in slot i % 3, so K_{j+1} is in flight while
            // tile j is being worked on
            for (int i = 0; i < 2 * n_kv; ++i) {
                const int slot = i % KV_SLOTS;
                const uint32_t par = (i / KV_SLOTS) & 1;
                if (!ptx::mbar_wait(&kv_empty[slot], par ^ 1)) {
                    atomicExch(args.status, DEV_TIMEOUT_ATTN);
                    break;
                }
                ptx::mbar_expect_tx(&kv_full[slot], TILE_BYTES);
                ptx::tma_load_4d(skv + slot * TILE_BYTES, (i & 1) ? &tmap_v : &tmap_k, &kv_full[slot], 0, (i >> 1) * KT, head,
                                 batch);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (ptx::elect_one()) {
            constexpr uint32_t IDESC_S = ptx::make_idesc_f16(128, KT, 0, 0);  // Q, K both K-major
            constexpr uint32_t IDESC_O = ptx::make_idesc_f16(128, HD, 0, 1);  // P K-major, V MN-major
            const uint32_t q_addr = ptx::smem_u32(sq), kv_addr = ptx::smem_u32(skv), p_addr = ptx::smem_u32(sp);
            bool ok = ptx::mbar_wait(q_full, 0);
            if (!ok) atomicExch(args.status, DEV_TIMEOUT_ATTN);
            for (int j = 0; ok && j < n_kv; ++j) {
                const uint32_t par = j & 1;
                // S_j = Q K_j^T
                const int ik = 2 * j, sk_ = ik % KV_SLOTS;
                if (!ptx::mbar_wait(&kv_full[sk_], (ik / KV_SLOTS) & 1)) {
                    atomicExch(args.status, DEV_TIMEOUT_ATTN);
                    break;
                }
                ptx::tc_fence_after();
                const uint32_t k_addr = kv_addr + sk_ * TILE_BYTES;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint64_t a = ptx::make_smem_desc_sw128(q_addr + kk * 32, 16, 1024);
                    const uint64_t b = ptx::make_smem_desc_sw128(k_addr + kk * 32, 16, 1024);
                    ptx::mma_f16_ss(tmem_s, a, b, IDESC_S, kk != 0 ? 1u : 0u);
                }
                ptx::mma_commit(s_full);
                ptx::mma_commit(&kv_empty[sk_]);
                // O_j = P_j V_j
                const int iv = 2 * j + 1, sv_ = iv % KV_SLOTS;
                if (!ptx::mbar_wait(p_full, par) || !ptx::mbar_wait(&kv_full[sv_], (iv / KV_SLOTS) & 1)) {
                    atomicExch(args.status, DEV_TIMEOUT_ATTN);
                    break;
                }
                ptx::tc_fence_after();
                const uint32_t v_addr = kv_addr + sv_ * TILE_BYTES;
#pragma unroll
                for (int kk = 0; kk < KT / 16; ++kk) {
                    // P: atom kk / 4 (64 keys each, 16 KB apart), 32 bytes per step inside the atom
                    const uint64_t a = ptx::make_smem_desc_sw128(p_addr + (kk >> 2) * (QT * 128) + (kk & 3) * 32, 16, 1024);
                    // V: 16 key rows of 128 bytes per step; 8-row groups 1024 bytes apart
                    const uint64_t b = ptx::make_smem_desc_sw128(v_addr + kk * 2048, 16, 1024);
                    ptx::mma_f16_ss(tmem_o, a, b, IDESC_O, kk != 0 ? 1u : 0u);
                }
                ptx::mma_commit(o_full);
                ptx::mma_commit(&kv_empty[sv_]);
            }
        }
    } else {
        // ------------------------------ softmax + output ------------------------------
        // Eight warps: warps q and q + 4 share TMEM lane quarter q; each thread owns one query row
        // and one half (64 keys) of the 128-key tile, and one half (32 columns) of the output row.
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        const int row = quarter * 32 + lane;  // row of the query tile == TMEM lane
        const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t s_addr = tmem_s + lane_off + half * 64;
        const uint32_t o_addr = tmem_o + lane_off + half * 32;
        uint8_t* p_row = sp + half * (QT * 128) + row * 128;  // this thread's 128-byte row of atom `half`
        float acc[HD / 2];
#pragma unroll
        for (int i = 0; i < HD / 2; ++i) acc[i] = 0.0f;
        float m_run = -INFINITY, l_run = 0.0f;
        const __half* mrow = args.mask ? args.mask + static_cast<int64_t>(batch) * args.seq_kv : nullptr;
        constexpr float LOG2E = 1.44269504088896340736f;
#ifdef B200ML_TRACE
        long long tr[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        long long tr_last = clock64();
#endif
        bool ok = true;
        for (int j = 0; j < n_kv; ++j) {
            const uint32_t par = j & 1;
            const int kv0 = j * KT + half * 64;  // first key of this thread's half
            if (!ptx::mbar_wait(s_full, par)) {
                if (lane == 0) atomicExch(args.status, DEV_TIMEOUT_ATTN);
                ok = false;
                break;
            }
            ptx::tc_fence_after();
            AT_MARK(0);  // waited for S
            // A tile is "plain" when every key is in range and there is no additive mask: the scale
            // then commutes with the maximum (one FMNMX per score) and P costs FFMA + EX2 + FADD.
            // The scores are read from TMEM once per pass, 32 columns at a time, to keep the
            // register footprint at two CTAs per SM.
            const bool plain = (j * KT + KT <= args.seq_kv) && mrow == nullptr && args.scale_log2 > 0.0f;
            float mx = -INFINITY;
            if (plain) {
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    uint32_t r[32];
                    ptx::tmem_ld_32x32b_x32(s_addr + u * 32, r);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
                }
            } else {
#pragma unroll 1
                for (int u = 0; u < 2; ++u) {
                    uint32_t r[32];
                    ptx::tmem_ld_32x32b_x32(s_addr + u * 32, r);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int kv = kv0 + u * 32 + i;
                        float v = __uint_as_float(r[i]) * args.scale_log2;
                        if (mrow && kv < args.seq_kv) v = fmaf(__half2float(__ldg(mrow + kv)), LOG2E, v);
                        if (kv >= args.seq_kv) v = -INFINITY;
                        mx = fmaxf(mx, v);
                    }
                }
            }
            if (plain) mx *= args.scale_log2;
            AT_MARK(1);  // pass 1
            // combine the two halves' maxima (the partner warp has the same lane quarter)
            xchg[(j & 1) * 256 + half * 128 + row] = mx;
            asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
            mx = fmaxf(fmaxf(mx, xchg[(j & 1) * 256 + (half ^ 1) * 128 + row]), m_run);
            AT_MARK(2);  // exchange
            const float m_safe = (mx == -INFINITY) ? 0.0f : mx;
            const float alpha = ex2(m_run - m_safe);  // 0 on the first tile
            float sum = 0.0f;
            if (plain) {
                const float neg_m = -m_safe;
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    uint32_t r[32];
                    ptx::tmem_ld_32x32b_x32(s_addr + u * 32, r);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        float p[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            p[i] = ex2(fmaf(__uint_as_float(r[g * 8 + i]), args.scale_log2, neg_m));
                            sum += p[i];
                        }
                        *reinterpret_cast<uint4*>(p_row + (((u * 4 + g) ^ (row & 7)) << 4)) = pack8(p);
                    }
                }
            } else {
#pragma unroll 1
                for (int u = 0; u < 2; ++u) {
                    uint32_t r[32];
                    ptx::tmem_ld_32x32b_x32(s_addr + u * 32, r);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        float p[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int kv = kv0 + u * 32 + g * 8 + i;
                            float v = __uint_as_float(r[g * 8 + i]) * args.scale_log2;
                            if (mrow && kv < args.seq_kv) v = fmaf(__half2float(__ldg(mrow + kv)), LOG2E, v);
                            p[i] = kv < args.seq_kv ? ex2(v - m_safe) : 0.0f;
                            sum += p[i];
                        }
                        *reinterpret_cast<uint4*>(p_row + (((u * 4 + g) ^ (row & 7)) << 4)) = pack8(p);
                    }
                }
            }
            AT_MARK(3);  // pass 2
            l_run = fmaf(l_run, alpha, sum);
            m_run = mx;
            ptx::fence_proxy_async_smem();  // P visible to the tensor core's shared-memory reads
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(p_full);
            AT_MARK(4);  // fence + arrive
            // fold this thread's half of O_j into the running output
            if (!ptx::mbar_wait(o_full, par)) {
                if (lane == 0) atomicExch(args.status, DEV_TIMEOUT_ATTN);
                ok = false;
                break;
            }
            ptx::tc_fence_after();
            AT_MARK(5);  // waited for O
            uint32_t ro[32];
            ptx::tmem_ld_32x32b_x32(o_addr, ro);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = fmaf(acc[i], alpha, __uint_as_float(ro[i]));
            ptx::tc_fence_before();
            AT_MARK(6);  // O accumulate
        }
#ifdef B200ML_TRACE
        if (threadIdx.x == 64 && blockIdx.x < 512) {
            for (int i = 0; i < 7; ++i) args.trace[blockIdx.x * 8 + i] = tr[i];
        }
#endif
        // the row sum is the sum of both halves' partial sums (they share every running maximum)
        xchg[512 + half * 128 + row] = l_run;
        asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
        const float l_tot = l_run + xchg[512 + (half ^ 1) * 128 + row];
        const int q = q0 + row;
        if (ok && q < args.seq_q) {
            const float inv = l_tot > 0.0f ? 1.0f / l_tot : 0.0f;
            __half* op = args.o + batch * args.o_stride_b + head * args.o_stride_h + static_cast<int64_t>(q) * args.o_stride_s +
                         half * 32;
            if ((reinterpret_cast<uintptr_t>(op) & 15) == 0) {
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    float v[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] = acc[g * 8 + i] * inv;
                    *reinterpret_cast<uint4*>(op + g * 8) = pack8(v);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) op[i] = __float2half_rn(acc[i] * inv);
            }
        }
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        if (*reinterpret_cast<volatile int32_t*>(args.status) != DEV_OK) {
            for (int i = 0; i < 200; ++i) __nanosleep(1000);
        }
        ptx::tmem_dealloc(tmem_base, AT_TMEM_COLS);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// {head_dim, seq, heads, batch} with a 64 x 128 box, 128-byte swizzle.
int make_qkv_tmap(const b200ml_ctx* ctx, CUtensorMap* out, const void* base, int64_t seq, int64_t heads, int64_t batch,
                  int64_t ss, int64_t sh, int64_t sb, const char* what) {
    if (!aligned16(base) || ss % 8 || (heads > 1 && sh % 8) || (batch > 1 && sb % 8))
        return fail(B200ML_ERR_UNSUPPORTED, "attention: %s is not 16-byte aligned in every stride", what);
    EncodeTiledFn fn = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled);
    if (!fn) return fail(B200ML_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const uint64_t dummy = static_cast<uint64_t>(ss) * 2 * static_cast<uint64_t>(seq);
    cuuint64_t dims[4] = {HD, (cuuint64_t)seq, (cuuint64_t)heads, (cuuint64_t)batch};
    cuuint64_t strides[3] = {(cuuint64_t)ss * 2, heads > 1 ? (cuuint64_t)sh * 2 : dummy, batch > 1 ? (cuuint64_t)sb * 2 : dummy};
    cuuint32_t box[4] = {HD, 128, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200ML_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)r);
    return B200ML_OK;
}

}  // namespace

int attention_f16(const b200ml_ctx* ctx, const b200ml_attention_params* p, cudaStream_t stream) {
    if (p->head_dim != HD)
        return fail(B200ML_ERR_UNSUPPORTED, "attention: head_dim %lld is not supported by the fused kernel (64 only)",
                    (long long)p->head_dim);
    if (p->mask && p->seq_kv >= (1ll << 31)) return fail(B200ML_ERR_INVALID, "attention: sequence too long");
    CUtensorMap tq, tk, tv;
    int rc = make_qkv_tmap(ctx, &tq, p->q, p->seq_q, p->heads, p->batch, p->q_stride_s, p->q_stride_h, p->q_stride_b, "Q");
    if (rc) return rc;
    rc = make_qkv_tmap(ctx, &tk, p->k, p->seq_kv, p->heads, p->batch, p->k_stride_s, p->k_stride_h, p->k_stride_b, "K");
    if (rc) return rc;
    rc = make_qkv_tmap(ctx, &tv, p->v, p->seq_kv, p->heads, p->batch, p->v_stride_s, p->v_stride_h, p->v_stride_b, "V");
    if (rc) return rc;
    AttnArgs a{};
    a.heads = (int32_t)p->heads;
    a.seq_q = (int32_t)p->seq_q;
    a.seq_kv = (int32_t)p->seq_kv;
    a.q_tiles = (int32_t)ceil_div(p->seq_q, QT);
    a.o_stride_b = p->o_stride_b;
    a.o_stride_h = p->o_stride_h;
    a.o_stride_s = p->o_stride_s;
    a.scale_log2 = p->scale * 1.44269504088896340736f;
    a.o = static_cast<__half*>(p->o);
    a.mask = static_cast<const __half*>(p->mask);
    a.status = ctx->status_dev;
    a.trace = static_cast<long long*>(ctx->workspace);
    const int64_t grid = p->batch * p->heads * a.q_tiles;
    B200ML_REQUIRE(grid < (1ll << 31), "attention: grid too large");
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        B200ML_CUDA(cudaFuncSetAttribute(attention_f16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM));
        configured[ctx->device & 63] = true;
    }
    attention_f16_kernel<<<(unsigned)grid, AT_THREADS, AT_SMEM, stream>>>(tq, tk, tv, a);
    return check_launch("attention_f16");
}

}  // namespace b200ml
