// Fused attention for fp16 tensors with head_dim 64: O = softmax(scale * Q K^T + mask) V.
//
// One CTA serves NC "chains" - NC tiles of 128 query rows of one (batch, head) - and NC x CTAs/SM
// is always 4 (four chains fill the 512 TMEM columns of an SM).  A chain is strictly serial
// (S_j -> softmax -> P_j -> O += P_j V_j, S_{j+1} -> ...); what keeps the SM busy is the other three
// chains on the same SM sub-partitions.  The chains of a CTA share the K / V tiles in shared memory,
// so K and V are fetched once per CTA.  Everything a chain exchanges with the tensor core lives in
// its 128 TMEM columns:
//   S [0,64)    scores of the current 64-key tile (fp32);
//   P           the first 32 columns of S, overwritten in place with the probabilities (fp16 pairs) -
//               the second product reads its A operand from TMEM, so P never touches shared memory;
//   O [64,128)  the running output (fp32), accumulated by the tensor core over all tiles.
// What bounds the kernel is the length of a chain's step, not a pipe: every hand-over (mbarrier,
// tcgen05.ld / st with their waits, tcgen05.commit) costs a few hundred cycles of latency, so the
// steps are as large as the registers allow (64 keys per thread and step) and as few as possible.
// Warps: 0 = TMA (Q tiles once, then K_j / V_j tiles straight from the caller's strided tensors, so
// Q/K/V may live inside a packed [T, 3H] projection output - no head split); 1 = the MMA issuer, one
// thread that serves whichever chain is ready (S_j = Q K_j^T, 128x64x64; O += P_j V_j, 128x64x64, V
// consumed MN-major exactly as TMA lays it down); then four softmax warps per chain, one query row
// per thread.
// O is rescaled only when a row maximum of the warp has grown by more than 2^8 since the last
// rescale (P then stays below 256, safe in fp16), which after the first tiles is rare; in the steady
// state the softmax threads never touch O.
// The scores never touch HBM: traffic is Q, K, V in and O out.
#include "common.cuh"
#include "ptx.cuh"
#include "epilogue.cuh"
#include "tensormap.cuh"
#include <math.h>

namespace b200ml {

namespace {

constexpr int QT = 128;          // query rows per chain
constexpr int KT = 64;           // keys per iteration
constexpr int HD = 64;           // head dimension
constexpr int Q_BYTES = QT * HD * 2;     // 16 KB
constexpr int KV_BYTES = KT * HD * 2;    // 8 KB: one K_j or V_j tile
constexpr int KV_SLOTS = 6;              // K and V tiles travel through one ring in the order the MMA warps consume them
constexpr int AT_BAR_BYTES = 512;
constexpr uint32_t CHAIN_COLS = 128;     // TMEM columns per chain
constexpr uint32_t O_COL = 64;
constexpr float RESCALE_STEP = 8.0f;     // log2 of the growth of a row maximum that forces a rescale
constexpr float M_NONE = -1.0e30f;       // running maximum of a row that has seen no finite score yet

template <int NC>
struct AttnCfg {
    static constexpr int THREADS = 32 * (2 + 4 * NC);
    static constexpr int CTAS_PER_SM = 4 / NC;
    static constexpr int SMEM = NC * Q_BYTES + KV_SLOTS * KV_BYTES + AT_BAR_BYTES + 1024;
    static constexpr uint32_t TMEM_COLS = CHAIN_COLS * NC;
};

struct AttnArgs {
    int32_t heads, seq_q, seq_kv, q_tiles, q_blocks;
    int64_t o_stride_b, o_stride_h, o_stride_s;
    float scale_log2;  // scale * log2(e)
    __half* o;
    const __half* mask;  // [batch, seq_kv] additive, or null
    int32_t* status;
};

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

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

template <int NC>
__global__ void __launch_bounds__(AttnCfg<NC>::THREADS, AttnCfg<NC>::CTAS_PER_SM)
attention_f16_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const AttnArgs args) {
    using Cfg = AttnCfg<NC>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sq = smem;                                  // NC Q tiles of 16 KB
    uint8_t* skv = smem + NC * Q_BYTES;                  // KV_SLOTS tiles of 4 KB
    uint64_t* bars = reinterpret_cast<uint64_t*>(skv + KV_SLOTS * KV_BYTES);
    uint64_t* q_full = bars;                    // [NC]
    uint64_t* kv_full = q_full + NC;            // [KV_SLOTS]
    uint64_t* kv_empty = kv_full + KV_SLOTS;    // [KV_SLOTS] one arrival per active chain
    uint64_t* s_full = kv_empty + KV_SLOTS;     // [NC] S of the chain holds a new tile, and every earlier product has finished
    uint64_t* p_full = s_full + NC;             // [NC] P is written (and O rescaled if it had to be)
    uint64_t* o_final = p_full + NC;            // [NC] every product of the chain has finished
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_final + NC);

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int qblk = blockIdx.x % args.q_blocks;
    const int bh = blockIdx.x / args.q_blocks;
    const int head = bh % args.heads;
    const int batch = bh / args.heads;
    const int n_kv = (args.seq_kv + KT - 1) / KT;
    const int left = args.q_tiles - qblk * NC;
    const int nc = left < NC ? left : NC;  // active chains of this CTA

    if (warp == 0 && lane == 0) {
        ptx::prefetch_tensormap(&tmap_q);
        ptx::prefetch_tensormap(&tmap_k);
        ptx::prefetch_tensormap(&tmap_v);
    }
    if (warp == 1) {
        if (lane == 0) {
            for (int i = 0; i < KV_SLOTS; ++i) {
                ptx::mbar_init(&kv_full[i], 1);
                ptx::mbar_init(&kv_empty[i], nc);
            }
            for (int c = 0; c < NC; ++c) {
                ptx::mbar_init(&q_full[c], 1);
                ptx::mbar_init(&s_full[c], 1);
                ptx::mbar_init(&p_full[c], 4);  // one arrival per softmax warp of the chain
                ptx::mbar_init(&o_final[c], 1);
            }
            ptx::fence_mbar_init();
        }
        __syncwarp();
        ptx::tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();  // everything above overlaps the previous kernel's tail

    // Order of consumption, which the ring follows: K_0, then for every j: V_j, K_{j+1} (if any).
    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (ptx::elect_one()) {
            for (int c = 0; c < nc; ++c) {
                ptx::mbar_expect_tx(&q_full[c], Q_BYTES);
                ptx::tma_load_4d(sq + c * Q_BYTES, &tmap_q, &q_full[c], 0, (qblk * NC + c) * QT, head, batch);
            }
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
                load(&tmap_v, j);
                if (ok && j + 1 < n_kv) load(&tmap_k, j + 1);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (one thread serves every chain) ------------------------------
        if (ptx::elect_one()) {
            constexpr uint32_t IDESC_S = ptx::make_idesc_f16(128, KT, 0, 0);  // Q, K both K-major
            constexpr uint32_t IDESC_O = ptx::make_idesc_f16(128, HD, 0, 1);  // P from TMEM, V MN-major
            const uint32_t kv_addr = ptx::smem_u32(skv);
            int next[NC];  // index of the chain's next O += P V
            int item[NC];  // the chain's position in the K / V ring
            bool ok = true;
            // S = Q K_t^T of chain c, from the ring item the chain has reached
            auto issue_s = [&](int c, int& it) {
                const int slot = it % KV_SLOTS;
                if (!ptx::mbar_wait(&kv_full[slot], (it / KV_SLOTS) & 1)) {
                    ok = false;
                    return;
                }
                ptx::tc_fence_after();
                const uint32_t q_addr = ptx::smem_u32(sq + c * Q_BYTES);
                const uint32_t k_addr = kv_addr + slot * KV_BYTES;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint64_t a = ptx::make_smem_desc_sw128(q_addr + kk * 32, 16, 1024);
                    const uint64_t b = ptx::make_smem_desc_sw128(k_addr + kk * 32, 16, 1024);
                    ptx::mma_f16_ss(tmem_base + c * CHAIN_COLS, a, b, IDESC_S, kk != 0 ? 1u : 0u);
                }
                ptx::mma_commit(&s_full[c]);
                ptx::mma_commit(&kv_empty[slot]);
                ++it;
            };
            int remaining = 0;
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                next[c] = 0;
                item[c] = 0;
                if (c < nc && ok) {
                    ok = ptx::mbar_wait(&q_full[c], 0);
                    if (ok && n_kv > 0) {
                        issue_s(c, item[c]);
                        ++remaining;
                    } else if (ok) {
                        ptx::mma_commit(&o_final[c]);
                    }
                }
            }
            // Serve whichever chain has published its P: O += P_j V_j, then S_{j+1} (the tensor core runs
            // this thread's instructions in order, so S_{j+1} lands only after P_j has been read).
            uint64_t t_last = ptx::global_timer_ns();
            uint32_t idle = 0;
            while (ok && remaining > 0) {
                bool progress = false;
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    if (c < nc && next[c] < n_kv && ok) {
                        const int j = next[c];
                        const int slot = item[c] % KV_SLOTS;
                        if (ptx::mbar_test_wait(&p_full[c], j & 1) && ptx::mbar_test_wait(&kv_full[slot], (item[c] / KV_SLOTS) & 1)) {
                            ptx::tc_fence_after();
                            const uint32_t chain = tmem_base + c * CHAIN_COLS;
                            const uint32_t v_addr = kv_addr + slot * KV_BYTES;
#pragma unroll
                            for (int kk = 0; kk < KT / 16; ++kk) {
                                // P: two keys per TMEM column, 8 columns per step; V: 16 key rows of 128 bytes per step
                                const uint64_t v = ptx::make_smem_desc_sw128(v_addr + kk * 2048, 16, 1024);
                                ptx::mma_f16_ts(chain + O_COL, chain + kk * 8, v, IDESC_O, (j != 0 || kk != 0) ? 1u : 0u);
                            }
                            ptx::mma_commit(&kv_empty[slot]);
                            ++item[c];
                            if (j + 1 < n_kv) {
                                issue_s(c, item[c]);
                            } else {
                                ptx::mma_commit(&o_final[c]);  // arrives when every product issued so far has finished
                                --remaining;
                            }
                            next[c] = j + 1;
                            progress = true;
                        }
                    }
                }
                if (progress) {
                    idle = 0;
                } else if ((++idle & 0x3ffu) == 0) {
                    const uint64_t now = ptx::global_timer_ns();
                    if (idle == 0x400u) t_last = now;  // first check of this idle stretch
                    if (now - t_last > ptx::kWaitLimitNs) ok = false;
                }
            }
            if (!ok) atomicExch(args.status, DEV_TIMEOUT_ATTN);
        }
    } else {
        // ------------------------------ softmax + output ------------------------------
        const int c = (warp - 2) >> 2;  // chain
        const int quarter = warp & 3;         // the TMEM lanes this warp may touch
        if (c < nc) {
            const int row = quarter * 32 + lane;  // row of the query tile == TMEM lane
            const uint32_t chain = tmem_base + c * CHAIN_COLS + (static_cast<uint32_t>(quarter * 32) << 16);
            const uint32_t o_addr = chain + O_COL;
            float m_used = M_NONE, l_run = 0.0f;
            const __half* mrow = args.mask ? args.mask + static_cast<int64_t>(batch) * args.seq_kv : nullptr;
            constexpr float LOG2E = 1.44269504088896340736f;
            bool ok = true;
            for (int j = 0; j < n_kv; ++j) {
                const int kv0 = j * KT;
                ok = __all_sync(0xffffffffu, ptx::mbar_wait(&s_full[c], j & 1));
                if (!ok) break;
                ptx::tc_fence_after();
                // A tile is "plain" when every key is in range and there is no additive mask: the scale then
                // commutes with the maximum (one FMNMX per two scores) and P costs FFMA + EX2 + FADD per score.
                const bool plain = (kv0 + KT <= args.seq_kv) && mrow == nullptr && args.scale_log2 > 0.0f;
                uint32_t r[2][32];
                ptx::tmem_ld_32x32b_x32(chain, r[0]);
                ptx::tmem_ld_32x32b_x32(chain + 32, r[1]);
                ptx::tmem_ld_wait();
                float mx;
                if (plain) {
                    float mx0 = max3(__uint_as_float(r[0][0]), __uint_as_float(r[0][1]), __uint_as_float(r[0][2]));
                    float mx1 = max3(__uint_as_float(r[1][0]), __uint_as_float(r[1][1]), __uint_as_float(r[1][2]));
#pragma unroll
                    for (int i = 3; i < 31; i += 2) {
                        mx0 = max3(mx0, __uint_as_float(r[0][i]), __uint_as_float(r[0][i + 1]));
                        mx1 = max3(mx1, __uint_as_float(r[1][i]), __uint_as_float(r[1][i + 1]));
                    }
                    mx = max3(mx0, mx1, fmaxf(__uint_as_float(r[0][31]), __uint_as_float(r[1][31]))) * args.scale_log2;
                } else {
                    // store the scaled, masked score back into the register it came from
                    mx = -INFINITY;
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
                if (__any_sync(0xffffffffu, mx > m_used + RESCALE_STEP)) {
                    const float m_new = fmaxf(m_used, mx);
                    const float f = ex2(m_used - m_new);  // 0 for a row that had no finite score so far
                    l_run *= f;
                    m_used = m_new;
                    if (j >= 1) {
                        // O is at rest: S_j arrived, so every earlier product of the chain has finished
#pragma unroll 1
                        for (int q = 0; q < HD / 16; ++q) {
                            uint32_t ro[16];
                            ptx::tmem_ld_32x32b_x16(o_addr + q * 16, ro);
                            ptx::tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 16; ++i) ro[i] = __float_as_uint(__uint_as_float(ro[i]) * f);
                            ptx::tmem_st_32x32b_x16(o_addr + q * 16, ro);
                        }
                    }
                }
                const float c_mul = plain ? args.scale_log2 : 1.0f;
                const float neg_m = -m_used;
                // all 64 exponentials first, nothing that depends on them in between: the special-function
                // unit then runs back to back; sums and fp16 packing follow
#pragma unroll
                for (int u = 0; u < 2; ++u)
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        r[u][i] = __float_as_uint(ex2(fmaf(__uint_as_float(r[u][i]), c_mul, neg_m)));
                float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                uint32_t pk[32];
#pragma unroll
                for (int u = 0; u < 2; ++u)
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        const float p0 = __uint_as_float(r[u][i]), p1 = __uint_as_float(r[u][i + 1]);
                        const float p2 = __uint_as_float(r[u][i + 2]), p3 = __uint_as_float(r[u][i + 3]);
                        sum[0] += p0;
                        sum[1] += p1;
                        sum[2] += p2;
                        sum[3] += p3;
                        pk[u * 16 + i / 2] = pack_half2(p0, p1);
                        pk[u * 16 + i / 2 + 1] = pack_half2(p2, p3);
                    }
                l_run += (sum[0] + sum[1]) + (sum[2] + sum[3]);
                ptx::tmem_st_32x32b_x32(chain, pk);  // P_j over the scores it came from
                ptx::tmem_st_wait();
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&p_full[c]);
            }
            if (!ok && lane == 0) atomicExch(args.status, DEV_TIMEOUT_ATTN);
            const bool done = __all_sync(0xffffffffu, ptx::mbar_wait(&o_final[c], 0));
            if (!done && lane == 0) atomicExch(args.status, DEV_TIMEOUT_ATTN);
            ptx::tc_fence_after();
            const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
            const int q = (qblk * NC + c) * QT + row;
            const bool store = ok && done && n_kv >= 1 && q < args.seq_q;
            __half* op = args.o + batch * args.o_stride_b + head * args.o_stride_h + static_cast<int64_t>(q) * args.o_stride_s;
            const bool vec = (reinterpret_cast<uintptr_t>(op) & 15) == 0;
#pragma unroll
            for (int h = 0; h < HD / 32; ++h) {
                uint32_t x[32];
                ptx::tmem_ld_32x32b_x32(o_addr + h * 32, x);  // every lane loads; only the stores are guarded
                ptx::tmem_ld_wait();
                if (store) {
                    if (vec) {
#pragma unroll
                        for (int g8 = 0; g8 < 4; ++g8) {
                            float v[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(x[g8 * 8 + i]) * inv;
                            *reinterpret_cast<uint4*>(op + h * 32 + g8 * 8) = pack8(v);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) op[h * 32 + i] = __float2half_rn(__uint_as_float(x[i]) * inv);
                    }
                }
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
        ptx::tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}


// {head_dim, seq, heads, batch} with a 64 x box_rows box, 128-byte swizzle.
int make_qkv_tmap(const b200ml_ctx* ctx, CUtensorMap* out, const void* base, int64_t seq, int64_t heads, int64_t batch,
                  int64_t ss, int64_t sh, int64_t sb, int box_rows, const char* what) {
    if (!aligned16(base) || ss % 8 || (heads > 1 && sh % 8) || (batch > 1 && sb % 8))
        return fail(B200ML_ERR_UNSUPPORTED, "attention: %s is not 16-byte aligned in every stride", what);
    if (!ctx->encode_tiled) return fail(B200ML_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const uint64_t dummy = static_cast<uint64_t>(ss) * 2 * static_cast<uint64_t>(seq);
    cuuint64_t dims[4] = {HD, (cuuint64_t)seq, (cuuint64_t)heads, (cuuint64_t)batch};
    cuuint64_t strides[3] = {(cuuint64_t)ss * 2, heads > 1 ? (cuuint64_t)sh * 2 : dummy, batch > 1 ? (cuuint64_t)sb * 2 : dummy};
    cuuint32_t box[4] = {HD, (cuuint32_t)box_rows, 1, 1};
    CUresult r = encode_tiled_cached(ctx, out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, base, dims, strides, box);
    if (r != CUDA_SUCCESS) return fail(B200ML_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)r);
    return B200ML_OK;
}

template <int NC>
int launch_attention(const b200ml_ctx* ctx, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, AttnArgs& a,
                     int64_t bh, cudaStream_t stream) {
    using Cfg = AttnCfg<NC>;
    a.q_blocks = (a.q_tiles + NC - 1) / NC;
    const int64_t grid = bh * a.q_blocks;
    B200ML_REQUIRE(grid < (1ll << 31), "attention: grid too large");
    auto kernel = attention_f16_kernel<NC>;
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        B200ML_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM));
        B200ML_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
        configured[ctx->device & 63] = true;
    }
    B200ML_CUDA(launch_pdl(kernel, dim3((unsigned)grid), dim3(Cfg::THREADS), Cfg::SMEM, stream, tq, tk, tv, a));
    return check_launch("attention_f16");
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
    // chains per CTA: as many query tiles of one (batch, head) as there are, up to four
    const int64_t bh = p->batch * p->heads;
    if (a.q_tiles >= 3) return launch_attention<4>(ctx, tq, tk, tv, a, bh, stream);
    if (a.q_tiles == 2) return launch_attention<2>(ctx, tq, tk, tv, a, bh, stream);
    return launch_attention<1>(ctx, tq, tk, tv, a, bh, stream);
}

}  // namespace b200ml
