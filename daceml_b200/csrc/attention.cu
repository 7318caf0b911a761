// Fused attention for fp16 tensors with head_dim 64: O = softmax(scale * Q K^T + mask) V.
//
// One CTA per (batch, head, 128 query rows).  A CTA is small on purpose - 192 threads, 128 TMEM
// columns, ~54 KB of shared memory - so that FOUR of them share an SM: the softmax of one tile is a
// chain of dependent steps (TMEM load, row maximum, exponentials, publish), and what hides that
// latency is other CTAs' chains on the same SM sub-partition.  Per 32-key tile:
//   warp 0   TMA loads of Q (once) and of the K_j / V_j tiles straight from the caller's strided
//            tensors (so Q/K/V may live inside a packed [T, 3H] projection output - no head split);
//   warp 1   tcgen05.mma S_j = Q K_j^T (128x32x64) into one of two S buffers in TMEM, and
//            O += P_j V_j (128x64x32) into the accumulator in TMEM; V is consumed MN-major exactly as
//            TMA lays it down - no transpose;
//   warps 2-5  one query row per thread: read S_j from TMEM, online softmax in the log2 domain, write
//            P_j (fp16) into shared memory in the 128-byte-swizzled K-major layout the MMA reads (tiles
//            alternate between the two halves of the 128-byte rows).
// O stays in TMEM for the whole CTA.  It is rescaled only when a row maximum of the warp has grown by
// more than 2^8 since the last rescale (P then stays below 256, safe in fp16), which after the first
// tiles is rare; in the steady state the softmax threads never touch O.
// The scores never touch HBM: traffic is Q, K, V in and O out.
#include "common.cuh"
#include "ptx.cuh"
#include "epilogue.cuh"
#include <math.h>

namespace b200ml {

namespace {

constexpr int AT_THREADS = 192;  // TMA warp, MMA warp, four softmax warps (one query row per thread)
constexpr int AT_CTAS_PER_SM = 4;
constexpr int QT = 128;          // query rows per CTA
constexpr int KT = 32;           // keys per iteration
constexpr int HD = 64;           // head dimension
constexpr int Q_BYTES = QT * HD * 2;     // 16 KB
constexpr int KV_BYTES = KT * HD * 2;    // 4 KB: one K_j or V_j tile
constexpr int P_BYTES = QT * 128;        // 16 KB: rows of 128 bytes = two tiles of 32 keys side by side
constexpr int KV_SLOTS = 5;              // K and V tiles travel through one ring in the order the MMA warp consumes them
constexpr int AT_SMEM = Q_BYTES + KV_SLOTS * KV_BYTES + P_BYTES + 256 + 1024;
constexpr uint32_t AT_TMEM_COLS = 128;   // S_0 [0,32), S_1 [32,64), O [64,128)
constexpr uint32_t O_COL = 64;
constexpr float RESCALE_STEP = 8.0f;     // log2 of the growth of a row maximum that forces a rescale
constexpr float M_NONE = -1.0e30f;       // running maximum of a row that has seen no finite score yet

struct AttnArgs {
    int32_t heads, seq_q, seq_kv, q_tiles;
    int64_t o_stride_b, o_stride_h, o_stride_s;
    float scale_log2;  // scale * log2(e)
    __half* o;
    const __half* mask;  // [batch, seq_kv] additive, or null
    int32_t* status;
    long long* trace;  // per-CTA cycle counters, only written when built with B200ML_TRACE
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

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__global__ void __launch_bounds__(AT_THREADS, AT_CTAS_PER_SM)
attention_f16_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const AttnArgs args) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sq = smem;
    uint8_t* skv = smem + Q_BYTES;                       // KV_SLOTS tiles of 4 KB
    uint8_t* sp = skv + KV_SLOTS * KV_BYTES;             // P: 128 rows of 128 bytes (1024-byte aligned: 16 KB + 5 * 4 KB)
    uint64_t* bars = reinterpret_cast<uint64_t*>(sp + P_BYTES);
    uint64_t* q_full = bars + 0;
    uint64_t* kv_full = bars + 1;               // [KV_SLOTS]
    uint64_t* kv_empty = kv_full + KV_SLOTS;    // [KV_SLOTS]
    uint64_t* s_full = kv_empty + KV_SLOTS;     // [2] S_b holds a new tile
    uint64_t* s_free = s_full + 2;              // [2] the softmax warps have S_b in registers
    uint64_t* p_full = s_free + 2;              // [2] P half b is written (and O rescaled if it had to be)
    uint64_t* o_full = p_full + 2;              // [2] O += P_b V finished: P half b may be overwritten
    uint64_t* o_final = o_full + 2;             // every product of this CTA has finished
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_final + 1);

    pdl_launch_dependents();
#ifdef B200ML_TRACE
    const long long tr_entry = clock64();
#endif
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
                ptx::mbar_init(&s_free[i], 4);  // one arrival per softmax warp
                ptx::mbar_init(&p_full[i], 4);
                ptx::mbar_init(&o_full[i], 1);
            }
            ptx::mbar_init(o_final, 1);
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

    // Order of consumption, which the ring follows: K_0, K_1, then for every j: K_{j+2} (if any), V_j.
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
            if (ok && n_kv > 1) load(&tmap_k, 1);
            for (int j = 0; ok && j < n_kv; ++j) {
                if (j + 2 < n_kv) load(&tmap_k, j + 2);
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
#ifdef B200ML_TRACE
            if (blockIdx.x < 512) args.trace[blockIdx.x * 20 + 10] = clock64() - tr_entry;
#endif
            bool ok = ptx::mbar_wait(q_full, 0);
            if (!ok) atomicExch(args.status, DEV_TIMEOUT_ATTN);
#ifdef B200ML_TRACE
            if (blockIdx.x < 512) args.trace[blockIdx.x * 20 + 11] = clock64() - tr_entry;
#endif
            // S_t = Q K_t^T into S buffer t & 1
#ifdef B200ML_TRACE
            long long mw[4] = {0, 0, 0, 0};
#define MW_T0() const long long _w0 = clock64()
#define MW_ADD(i) mw[i] += clock64() - _w0
#else
#define MW_T0()
#define MW_ADD(i)
#endif
            auto issue_s = [&](int t) {
                const int slot = item % KV_SLOTS;
                MW_T0();
                const bool got = ptx::mbar_wait(&kv_full[slot], (item / KV_SLOTS) & 1);
                MW_ADD(1);
                if (!got) {
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
            if (ok && n_kv > 1) issue_s(1);
            for (int j = 0; ok && j < n_kv; ++j) {
                const int b = j & 1;
                const uint32_t use = (j >> 1) & 1;  // parity of the buffer's use counter
                if (j + 2 < n_kv) {
                    // S_j is in registers: its buffer takes the tile after next
                    MW_T0();
                    const bool got = ptx::mbar_wait(&s_free[b], use);
                    MW_ADD(0);
                    if (!got) {
                        atomicExch(args.status, DEV_TIMEOUT_ATTN);
                        break;
                    }
                    issue_s(j + 2);
                    if (!ok) break;
                }
                // O += P_j V_j
                const int slot = item % KV_SLOTS;
                bool got;
                {
                    MW_T0();
                    got = ptx::mbar_wait(&p_full[b], use);
                    MW_ADD(2);
                }
                {
                    MW_T0();
                    got = got && ptx::mbar_wait(&kv_full[slot], (item / KV_SLOTS) & 1);
                    MW_ADD(3);
                }
                if (!got) {
                    atomicExch(args.status, DEV_TIMEOUT_ATTN);
                    break;
                }
                ptx::tc_fence_after();
                const uint32_t v_addr = kv_addr + slot * KV_BYTES;
#pragma unroll
                for (int kk = 0; kk < KT / 16; ++kk) {
                    // P: 32 bytes per 16-key step inside the 128-byte swizzle row; V: 16 key rows of 128 bytes per step
                    const uint64_t a = ptx::make_smem_desc_sw128(p_addr + (b * 2 + kk) * 32, 16, 1024);
                    const uint64_t v = ptx::make_smem_desc_sw128(v_addr + kk * 2048, 16, 1024);
                    ptx::mma_f16_ss(tmem_base + O_COL, a, v, IDESC_O, (j != 0 || kk != 0) ? 1u : 0u);
                }
                ptx::mma_commit(&o_full[b]);
                ptx::mma_commit(&kv_empty[slot]);
                ++item;
            }
            ptx::mma_commit(o_final);  // arrives when every product issued above has finished
#ifdef B200ML_TRACE
            if (blockIdx.x < 512) for (int i = 0; i < 4; ++i) args.trace[blockIdx.x * 20 + 14 + i] = mw[i];
#endif
        }
    } else {
        // ------------------------------ softmax + output ------------------------------
        const int quarter = warp & 3;    // the TMEM lanes this warp may touch
        const int row = quarter * 32 + lane;  // row of the query tile == TMEM lane
        const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t o_addr = tmem_base + O_COL + lane_off;
        uint8_t* p_row = sp + row * 128;
        float m_used = M_NONE, l_run = 0.0f;
        const __half* mrow = args.mask ? args.mask + static_cast<int64_t>(batch) * args.seq_kv : nullptr;
        constexpr float LOG2E = 1.44269504088896340736f;
        bool ok = true;
#ifdef B200ML_TRACE
        long long tr[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        long long tr_last = clock64();
        const long long tr_begin = tr_last;
#endif
        for (int j = 0; j < n_kv; ++j) {
            const int kv0 = j * KT;
            const int b = j & 1;
            const uint32_t use = (j >> 1) & 1;
            ok = __all_sync(0xffffffffu, ptx::mbar_wait(&s_full[b], use));
            if (!ok) break;
            ptx::tc_fence_after();
            AT_MARK(0);
#ifdef B200ML_TRACE
            if (j == 0 && threadIdx.x == 64 && blockIdx.x < 512) args.trace[blockIdx.x * 20 + 12] = clock64() - tr_entry;
#endif
            // A tile is "plain" when every key is in range and there is no additive mask: the scale then
            // commutes with the maximum (one FMNMX per two scores) and P costs FFMA + EX2 + FADD per score.
            const bool plain = (kv0 + KT <= args.seq_kv) && mrow == nullptr && args.scale_log2 > 0.0f;
            uint32_t r[32];
            ptx::tmem_ld_32x32b_x32(tmem_base + b * KT + lane_off, r);
            ptx::tmem_ld_wait();
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&s_free[b]);
            AT_MARK(1);
            float mx;
            if (plain) {
                float mx0 = max3(__uint_as_float(r[0]), __uint_as_float(r[1]), __uint_as_float(r[2]));
                float mx1 = max3(__uint_as_float(r[3]), __uint_as_float(r[4]), __uint_as_float(r[5]));
#pragma unroll
                for (int i = 6; i < 30; i += 4) {
                    mx0 = max3(mx0, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
                    mx1 = max3(mx1, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
                }
                mx = max3(mx0, mx1, fmaxf(__uint_as_float(r[30]), __uint_as_float(r[31]))) * args.scale_log2;
            } else {
                // store the scaled, masked score back into the register it came from
                mx = -INFINITY;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int kv = kv0 + i;
                    float v = __uint_as_float(r[i]) * args.scale_log2;
                    if (mrow && kv < args.seq_kv) v = fmaf(__half2float(__ldg(mrow + kv)), LOG2E, v);
                    if (kv >= args.seq_kv) v = -INFINITY;
                    r[i] = __float_as_uint(v);
                    mx = fmaxf(mx, v);
                }
            }
            AT_MARK(2);
            if (j >= 2) {
                // the product of the tile before last has finished reading this half of P
                ok = __all_sync(0xffffffffu, ptx::mbar_wait(&o_full[b], use ^ 1));
                if (!ok) break;
            }
            AT_MARK(3);
            if (__any_sync(0xffffffffu, mx > m_used + RESCALE_STEP)) {
                const float m_new = fmaxf(m_used, mx);
                const float f = ex2(m_used - m_new);  // 0 for a row that had no finite score so far
                l_run *= f;
                m_used = m_new;
                if (j >= 1) {
                    // O must be at rest: wait for the product of the previous tile as well
                    ok = __all_sync(0xffffffffu, ptx::mbar_wait(&o_full[b ^ 1], ((j - 1) >> 1) & 1));
                    if (!ok) break;
                    ptx::tc_fence_after();
#pragma unroll 1
                    for (int c = 0; c < HD / 16; ++c) {
                        uint32_t ro[16];
                        ptx::tmem_ld_32x32b_x16(o_addr + c * 16, ro);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i) ro[i] = __float_as_uint(__uint_as_float(ro[i]) * f);
                        ptx::tmem_st_32x32b_x16(o_addr + c * 16, ro);
                    }
                    ptx::tmem_st_wait();
                }
#ifdef B200ML_TRACE
                tr[7] += 1;
#endif
            }
            AT_MARK(4);
            float sum0 = 0.0f, sum1 = 0.0f;
            const float c_mul = plain ? args.scale_log2 : 1.0f;
            const float neg_m = -m_used;
#pragma unroll
            for (int q8 = 0; q8 < 4; ++q8) {
                float p[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) p[i] = ex2(fmaf(__uint_as_float(r[q8 * 8 + i]), c_mul, neg_m));
                sum0 += (p[0] + p[1]) + (p[2] + p[3]);
                sum1 += (p[4] + p[5]) + (p[6] + p[7]);
                *reinterpret_cast<uint4*>(p_row + (((b * 4 + q8) ^ (row & 7)) << 4)) = pack8(p);
            }
            l_run += sum0 + sum1;
            AT_MARK(5);
            ptx::fence_proxy_async_smem();  // P visible to the tensor core's shared-memory reads
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&p_full[b]);
            AT_MARK(6);
        }
#ifdef B200ML_TRACE
        if (threadIdx.x == 64 && blockIdx.x < 512) {
            long long* t = args.trace + blockIdx.x * 20;
            for (int i = 0; i < 8; ++i) t[i] = tr[i];
            t[8] = clock64() - tr_begin;
            t[9] = tr_begin - tr_entry;
        }
#endif
        if (!ok && lane == 0) atomicExch(args.status, DEV_TIMEOUT_ATTN);
        const bool done = __all_sync(0xffffffffu, ptx::mbar_wait(o_final, 0));
        if (!done && lane == 0) atomicExch(args.status, DEV_TIMEOUT_ATTN);
        ptx::tc_fence_after();
        const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
        const int q = q0 + row;
        const bool store = ok && done && n_kv >= 1 && q < args.seq_q;
        __half* op = args.o + batch * args.o_stride_b + head * args.o_stride_h + static_cast<int64_t>(q) * args.o_stride_s;
        const bool vec = (reinterpret_cast<uintptr_t>(op) & 15) == 0;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
            uint32_t x[32];
            ptx::tmem_ld_32x32b_x32(o_addr + c * 32, x);  // every lane loads; only the stores are guarded
            ptx::tmem_ld_wait();
            if (store) {
                if (vec) {
#pragma unroll
                    for (int g8 = 0; g8 < 4; ++g8) {
                        float v[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(x[g8 * 8 + i]) * inv;
                        *reinterpret_cast<uint4*>(op + c * 32 + g8 * 8) = pack8(v);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) op[c * 32 + i] = __float2half_rn(__uint_as_float(x[i]) * inv);
                }
            }
        }
    }

    ptx::tc_fence_before();
    __syncthreads();
#ifdef B200ML_TRACE
    if (threadIdx.x == 64 && blockIdx.x < 512) args.trace[blockIdx.x * 20 + 13] = clock64() - tr_entry;
#endif
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
        B200ML_CUDA(cudaFuncSetAttribute(attention_f16_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
        configured[ctx->device & 63] = true;
    }
    B200ML_CUDA(launch_pdl(attention_f16_kernel, dim3((unsigned)grid), dim3(AT_THREADS), AT_SMEM, stream, tq, tk, tv, a));
    return check_launch("attention_f16");
}

}  // namespace b200ml
