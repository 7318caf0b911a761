// Fused attention for fp16 tensors with head_dim 64: O = softmax(scale * Q K^T + mask) V.
//
// One CTA per (batch, head, 128 query rows); two CTAs share an SM.  Per 64-key tile:
//   warp 0   TMA loads of Q (once) and of the K_j / V_j tiles straight from the caller's strided
//            tensors (so Q/K/V may live inside a packed [T, 3H] projection output - no head split);
//   warp 1   tcgen05.mma S_j = Q K_j^T (128x64x64) into TMEM, O_j = P_j V_j (128x64x64);
//            V is consumed MN-major exactly as TMA lays it down - no transpose;
//   warps 2-5  one query row per thread: read S_j from TMEM, online softmax in the log2 domain,
//            write P_j (fp16) into shared memory in the 128-byte-swizzled K-major layout the MMA
//            reads, then fold O_{j-1} into the fp32 running output held in registers.
// The scores never touch HBM: traffic is Q, K, V in and O out.
#include "common.cuh"
#include "ptx.cuh"
#include "epilogue.cuh"
#include <math.h>

namespace b200ml {

namespace {

constexpr int AT_THREADS = 192;  // TMA warp, MMA warp, four softmax warps (one query row per thread)
constexpr int QT = 128;          // query rows per CTA
constexpr int KT = 64;           // keys per iteration
constexpr int HD = 64;           // head dimension
constexpr int Q_BYTES = QT * HD * 2;     // 16 KB
constexpr int KV_BYTES = KT * HD * 2;    // 8 KB: one K_j or V_j tile
constexpr int P_BYTES = QT * KT * 2;     // 16 KB: one 64-key swizzle atom
constexpr int KV_SLOTS = 4;              // K and V tiles travel through one ring in the order the MMA warp consumes them
constexpr int AT_SMEM = Q_BYTES + KV_SLOTS * KV_BYTES + 2 * P_BYTES + 256 + 1024;
constexpr uint32_t AT_TMEM_COLS = 256;   // S_even [0,64), S_odd [64,128), O_even [128,192), O_odd [192,256)

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

// Everything the softmax warps and the tensor core exchange is double-buffered (S and O in TMEM, P in
// shared memory), so S_{j+1} = Q K_{j+1}^T and O_{j-1} = P_{j-1} V_{j-1} run on the tensor core while
// the softmax of tile j runs on the SIMT pipes.  The fold of O_{j-1} into the running output is
// deferred by one tile for the same reason.
__global__ void __launch_bounds__(AT_THREADS, 2)
attention_f16_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const AttnArgs args) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sq = smem;
    uint8_t* skv = smem + Q_BYTES;                       // KV_SLOTS tiles of 8 KB
    uint8_t* sp = skv + KV_SLOTS * KV_BYTES;             // two P buffers
    uint64_t* bars = reinterpret_cast<uint64_t*>(sp + 2 * P_BYTES);
    uint64_t* q_full = bars + 0;
    uint64_t* kv_full = bars + 1;               // [KV_SLOTS]
    uint64_t* kv_empty = kv_full + KV_SLOTS;    // [KV_SLOTS]
    uint64_t* s_full = kv_empty + KV_SLOTS;     // [2]
    uint64_t* p_full = s_full + 2;              // [2]
    uint64_t* o_full = p_full + 2;              // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 2);

    pdl_launch_dependents();
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
            for (int i = 0; i < 2; ++i) {
                ptx::mbar_init(&s_full[i], 1);
                ptx::mbar_init(&p_full[i], 4);  // one arrival per softmax warp
                ptx::mbar_init(&o_full[i], 1);
            }
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
    pdl_wait();  // everything above overlaps the previous kernel's tail

    // The ring carries K_0, then for every j: K_{j+1} (if any), V_j -- the order of consumption.
    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (ptx::elect_one()) {
            ptx::mbar_expect_tx(q_full, Q_BYTES);
            ptx::tma_load_4d(sq, &tmap_q, q_full, 0, q0, head, batch);
            int item = 0;
            bool ok = true;
            auto load = [&](const CUtensorMap* map, int tile) {
                const int slot = item % KV_SLOTS;
                if (!ptx::mbar_wait(&kv_empty[slot], ((item / KV_SLOTS) & 1) ^ 1)) {
                    atomicExch(args.status, DEV_TIMEOUT_ATTN);
                    ok = false;
                    return;
                }
                ptx::mbar_expect_tx(&kv_full[slot], KV_BYTES);
                ptx::tma_load_4d(skv + slot * KV_BYTES, map, &kv_full[slot], 0, tile * KT, head, batch);
                ++item;
            };
            load(&tmap_k, 0);
            for (int j = 0; ok && j < n_kv; ++j) {
                if (j + 1 < n_kv) load(&tmap_k, j + 1);
                if (ok) load(&tmap_v, j);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (ptx::elect_one()) {
            constexpr uint32_t IDESC_S = ptx::make_idesc_f16(128, KT, 0, 0);  // Q, K both K-major
            constexpr uint32_t IDESC_O = ptx::make_idesc_f16(128, HD, 0, 1);  // P K-major, V MN-major
            const uint32_t q_addr = ptx::smem_u32(sq), kv_addr = ptx::smem_u32(skv), p_addr = ptx::smem_u32(sp);
            int item = 0;
            bool ok = ptx::mbar_wait(q_full, 0);
            if (!ok) atomicExch(args.status, DEV_TIMEOUT_ATTN);
            // S_t = Q K_t^T into S buffer t & 1; the buffer's previous tile was consumed before P_{t-2} was
            // published, which this thread has already waited for.
            auto issue_s = [&](int t) {
                const int slot = item % KV_SLOTS;
                if (!ptx::mbar_wait(&kv_full[slot], (item / KV_SLOTS) & 1)) {
                    atomicExch(args.status, DEV_TIMEOUT_ATTN);
                    ok = false;
                    return;
                }
                ptx::tc_fence_after();
                const uint32_t k_addr = kv_addr + slot * KV_BYTES;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint64_t a = ptx::make_smem_desc_sw128(q_addr + kk * 32, 16, 1024);
                    const uint64_t b = ptx::make_smem_desc_sw128(k_addr + kk * 32, 16, 1024);
                    ptx::mma_f16_ss(tmem_base + (t & 1) * KT, a, b, IDESC_S, kk != 0 ? 1u : 0u);
                }
                ptx::mma_commit(&s_full[t & 1]);
                ptx::mma_commit(&kv_empty[slot]);
                ++item;
            };
            if (ok) issue_s(0);
            for (int j = 0; ok && j < n_kv; ++j) {
                if (j + 1 < n_kv) issue_s(j + 1);
                if (!ok) break;
                // O_j = P_j V_j into O buffer j & 1 (its previous tile was folded before P_j was published)
                const int slot = item % KV_SLOTS;
                if (!ptx::mbar_wait(&p_full[j & 1], (j >> 1) & 1) || !ptx::mbar_wait(&kv_full[slot], (item / KV_SLOTS) & 1)) {
                    atomicExch(args.status, DEV_TIMEOUT_ATTN);
                    break;
                }
                ptx::tc_fence_after();
                const uint32_t v_addr = kv_addr + slot * KV_BYTES;
                const uint32_t pj_addr = p_addr + (j & 1) * P_BYTES;
#pragma unroll
                for (int kk = 0; kk < KT / 16; ++kk) {
                    // P: 32 bytes per 16-key step inside the 128-byte swizzle row; V: 16 key rows of 128 bytes per step
                    const uint64_t a = ptx::make_smem_desc_sw128(pj_addr + kk * 32, 16, 1024);
                    const uint64_t b = ptx::make_smem_desc_sw128(v_addr + kk * 2048, 16, 1024);
                    ptx::mma_f16_ss(tmem_base + 128 + (j & 1) * HD, a, b, IDESC_O, kk != 0 ? 1u : 0u);
                }
                ptx::mma_commit(&o_full[j & 1]);
                ptx::mma_commit(&kv_empty[slot]);
                ++item;
            }
        }
    } else {
        // ------------------------------ softmax + output ------------------------------
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;  // row of the query tile == TMEM lane
        const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
        float acc[HD];
#pragma unroll
        for (int i = 0; i < HD; ++i) acc[i] = 0.0f;
        float m_run = -INFINITY, l_run = 0.0f, alpha_prev = 0.0f;
        const __half* mrow = args.mask ? args.mask + static_cast<int64_t>(batch) * args.seq_kv : nullptr;
        constexpr float LOG2E = 1.44269504088896340736f;
#ifdef B200ML_TRACE
        long long tr[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        long long tr_last = clock64();
#endif
        bool ok = true;
        // folds O_t (finished by the tensor core) into the running output: acc = acc * alpha_t + O_t
        auto fold = [&](int t, float alpha) {
            if (!ptx::mbar_wait(&o_full[t & 1], (t >> 1) & 1)) {
                if (lane == 0) atomicExch(args.status, DEV_TIMEOUT_ATTN);
                ok = false;
                return;
            }
            ptx::tc_fence_after();
            AT_MARK(4);
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t ro[32];
                ptx::tmem_ld_32x32b_x32(tmem_base + 128 + (t & 1) * HD + lane_off + c * 32, ro);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[c * 32 + i] = fmaf(acc[c * 32 + i], alpha, __uint_as_float(ro[i]));
            }
            ptx::tc_fence_before();
            AT_MARK(5);
        };
        for (int j = 0; ok && j < n_kv; ++j) {
            const int kv0 = j * KT;
            const uint32_t s_addr = tmem_base + (j & 1) * KT + lane_off;
            uint8_t* p_row = sp + (j & 1) * P_BYTES + row * 128;
            if (!ptx::mbar_wait(&s_full[j & 1], (j >> 1) & 1)) {
                if (lane == 0) atomicExch(args.status, DEV_TIMEOUT_ATTN);
                ok = false;
                break;
            }
            ptx::tc_fence_after();
            AT_MARK(0);
            // A tile is "plain" when every key is in range and there is no additive mask: the scale then
            // commutes with the maximum (one FMNMX per score) and P costs FFMA + EX2 + FADD per score.
            const bool plain = (kv0 + KT <= args.seq_kv) && mrow == nullptr && args.scale_log2 > 0.0f;
            uint32_t r[2][32];
            ptx::tmem_ld_32x32b_x32(s_addr, r[0]);
            ptx::tmem_ld_32x32b_x32(s_addr + 32, r[1]);
            ptx::tmem_ld_wait();
            float mx = -INFINITY;
            if (plain) {
#pragma unroll
                for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fmaxf(__uint_as_float(r[0][i]), __uint_as_float(r[1][i])));
                mx *= args.scale_log2;
            } else {
                // store the scaled, masked score back into the register it came from
#pragma unroll
                for (int u = 0; u < 2; ++u)
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int kv = kv0 + u * 32 + i;
                        float v = __uint_as_float(r[u][i]) * args.scale_log2;
                        if (mrow && kv < args.seq_kv) v = fmaf(__half2float(__ldg(mrow + kv)), LOG2E, v);
                        if (kv >= args.seq_kv) v = -INFINITY;
                        r[u][i] = __float_as_uint(v);
                        mx = fmaxf(mx, v);
                    }
            }
            mx = fmaxf(mx, m_run);
            const float m_safe = (mx == -INFINITY) ? 0.0f : mx;
            const float alpha = ex2(m_run - m_safe);  // 0 on the first tile
            AT_MARK(1);
            float sum = 0.0f;
            const float c_mul = plain ? args.scale_log2 : 1.0f;
            const float neg_m = -m_safe;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    float p[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        p[i] = ex2(fmaf(__uint_as_float(r[u][g * 8 + i]), c_mul, neg_m));
                        sum += p[i];
                    }
                    *reinterpret_cast<uint4*>(p_row + (((u * 4 + g) ^ (row & 7)) << 4)) = pack8(p);
                }
            }
            l_run = fmaf(l_run, alpha, sum);
            m_run = mx;
            AT_MARK(2);
            ptx::fence_proxy_async_smem();  // P visible to the tensor core's shared-memory reads
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&p_full[j & 1]);
            AT_MARK(3);
            if (j >= 1) fold(j - 1, alpha_prev);
            alpha_prev = alpha;
        }
        if (ok && n_kv >= 1) fold(n_kv - 1, alpha_prev);
#ifdef B200ML_TRACE
        if (threadIdx.x == 64 && blockIdx.x < 512) {
            for (int i = 0; i < 7; ++i) args.trace[blockIdx.x * 8 + i] = tr[i];
        }
#endif
        const int q = q0 + row;
        if (ok && q < args.seq_q) {
            const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
            __half* op = args.o + batch * args.o_stride_b + head * args.o_stride_h + static_cast<int64_t>(q) * args.o_stride_s;
            if ((reinterpret_cast<uintptr_t>(op) & 15) == 0) {
#pragma unroll
                for (int g = 0; g < HD / 8; ++g) {
                    float v[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] = acc[g * 8 + i] * inv;
                    *reinterpret_cast<uint4*>(op + g * 8) = pack8(v);
                }
            } else {
#pragma unroll
                for (int i = 0; i < HD; ++i) op[i] = __float2half_rn(acc[i] * inv);
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

// {head_dim, seq, heads, batch} with a 64 x box_rows box, 128-byte swizzle.
int make_qkv_tmap(const b200ml_ctx* ctx, CUtensorMap* out, const void* base, int64_t seq, int64_t heads, int64_t batch,
                  int64_t ss, int64_t sh, int64_t sb, int box_rows, const char* what) {
    if (!aligned16(base) || ss % 8 || (heads > 1 && sh % 8) || (batch > 1 && sb % 8))
        return fail(B200ML_ERR_UNSUPPORTED, "attention: %s is not 16-byte aligned in every stride", what);
    EncodeTiledFn fn = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled);
    if (!fn) return fail(B200ML_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const uint64_t dummy = static_cast<uint64_t>(ss) * 2 * static_cast<uint64_t>(seq);
    cuuint64_t dims[4] = {HD, (cuuint64_t)seq, (cuuint64_t)heads, (cuuint64_t)batch};
    cuuint64_t strides[3] = {(cuuint64_t)ss * 2, heads > 1 ? (cuuint64_t)sh * 2 : dummy, batch > 1 ? (cuuint64_t)sb * 2 : dummy};
    cuuint32_t box[4] = {HD, (cuuint32_t)box_rows, 1, 1};
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
    int rc = make_qkv_tmap(ctx, &tq, p->q, p->seq_q, p->heads, p->batch, p->q_stride_s, p->q_stride_h, p->q_stride_b, QT, "Q");
    if (rc) return rc;
    rc = make_qkv_tmap(ctx, &tk, p->k, p->seq_kv, p->heads, p->batch, p->k_stride_s, p->k_stride_h, p->k_stride_b, KT, "K");
    if (rc) return rc;
    rc = make_qkv_tmap(ctx, &tv, p->v, p->seq_kv, p->heads, p->batch, p->v_stride_s, p->v_stride_h, p->v_stride_b, KT, "V");
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
    B200ML_CUDA(launch_pdl(attention_f16_kernel, dim3((unsigned)grid), dim3(AT_THREADS), AT_SMEM, stream, tq, tk, tv, a));
    return check_launch("attention_f16");
}

}  // namespace b200ml
