// The epilogue of the GEMM + LayerNorm kernels: everything after the last product of a CTA's 128 x 256 tile.
//   pass A   finish the GEMM epilogue in fp32 (alpha, bias, ReLU, residual), park the values in TMEM, accumulate
//            the row's sum and sum of squares;
//   exchange the CTAs that hold the other columns of the same rows read each other's per-row sums through
//            distributed shared memory, between two cluster barriers;
//   pass B   normalise, scale, shift, stage in shared memory, bulk tensor store.
// Called by every thread of the CTA (the cluster barriers need all of them); warps 2-9 do the work.
#pragma once

#include "gemm_common.cuh"

namespace b200ml {
namespace gemm {

struct LnArgs {
    GemmArgs g;
    const __half* gamma;
    const __half* beta;
    float eps;
    int32_t cluster;  // CTAs (or CTA pairs) per row block = N / 256
};

// Where the sixteen 32-row x 64-column residual tiles of a CTA sit in shared memory (tile t: epilogue warp t / 2,
// its 64-column half t % 2): the first `split` tiles in one freed pipeline stage, the rest in the next.
struct ResidualTiles {
    uint8_t* first;
    uint8_t* second;
    int split;
    bool present;
    __device__ __forceinline__ uint8_t* tile(int t) const { return t < split ? first + t * 4096 : second + (t - split) * 4096; }
};

// peers: the NPEERS cluster ranks peer_first + i * peer_step hold the same rows.  G: 32-column chunks in flight per
// warp (2 needs about 168 registers per thread, 1 about 96).
template <int NPEERS, int G>
__device__ __forceinline__ void layernorm_epilogue(const LnArgs& la, const CUtensorMap* tmap_c, uint32_t tmem_base,
                                                   uint8_t* out_stage, const ResidualTiles& res, float* red, float* stats,
                                                   uint64_t* tmem_full_bar, uint64_t* res_full_bar, int m0, int n0,
                                                   uint32_t peer_first, uint32_t peer_step, int warp, int lane) {
    const GemmArgs& args = la.g;
    bool epi_ok = true;
    const bool is_epi = warp >= 2;
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;           // columns [half * 128, half * 128 + 128) of this CTA's tile
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t t_base = tmem_base + half * 128 + (static_cast<uint32_t>(quarter * 32) << 16);
    const int col_base = n0 + half * 128;
    const float inv_n = 1.0f / static_cast<float>(args.n);
    float mean = 0.0f, rstd = 0.0f;

    // pass A: finish the GEMM epilogue in fp32, park the values in TMEM, accumulate the row's sum and sum of squares
    if (is_epi) {
        if (!ptx::mbar_wait(tmem_full_bar, 0)) {
            if (lane == 0) atomicExch(args.status, DEV_TIMEOUT_EPILOGUE);
            epi_ok = false;
        }
        ptx::tc_fence_after();
        float s1 = 0.0f, s2 = 0.0f;
        if (epi_ok) {
            const bool has_bias = (args.epilogue & B200ML_EPI_BIAS) && args.bias;
            const bool has_res = res.present;  // rows past M read the zeros the tensor map fills in
            if (has_res && !ptx::mbar_wait(res_full_bar, 0)) {
                if (lane == 0) atomicExch(args.status, DEV_TIMEOUT_EPILOGUE);
                epi_ok = false;
            }
            const bool relu = (args.epilogue & B200ML_EPI_RELU) != 0;
#pragma unroll 1
            for (int c = 0; c < 4; c += G) {
                uint32_t r[G][32];
                uint4 rb[G][4], rr[G][4];
#pragma unroll
                for (int u = 0; u < G; ++u) ptx::tmem_ld_32x32b_x32(t_base + (c + u) * 32, r[u]);
#pragma unroll
                for (int u = 0; u < G; ++u) {
                    const int col0 = col_base + (c + u) * 32;
                    if (has_bias) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) rb[u][g] = __ldg(reinterpret_cast<const uint4*>(args.bias + col0 + g * 8));
                    }
                    if (has_res) {
                        const uint8_t* tile_row = res.tile((warp - 2) * 2 + ((c + u) >> 1)) + lane * 128;
#pragma unroll
                        for (int g = 0; g < 4; ++g)
                            rr[u][g] = *reinterpret_cast<const uint4*>(tile_row + (((((c + u) & 1) * 4 + g) ^ (lane & 7)) << 4));
                    }
                }
                ptx::tmem_ld_wait();
#pragma unroll
                for (int u = 0; u < G; ++u) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        float b[8], q[8];
                        if (has_bias) unpack8(rb[u][g], b);
                        if (has_res) unpack8(rr[u][g], q);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            float v = args.alpha * __uint_as_float(r[u][g * 8 + j]);
                            if (has_bias) v = fmaf(args.bias_scale, b[j], v);
                            if (relu) v = fmaxf(v, 0.0f);
                            if (has_res) v = fmaf(args.residual_scale, q[j], v);
                            s1 += v;
                            s2 = fmaf(v, v, s2);
                            r[u][g * 8 + j] = __float_as_uint(v);
                        }
                    }
                    ptx::tmem_st_32x32b_x32(t_base + (c + u) * 32, r[u]);
                }
            }
            ptx::tmem_st_wait();
        }
        red[half * BM + row_in_tile] = s1;
        red[(2 + half) * BM + row_in_tile] = s2;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (half == 0) {
            stats[row_in_tile] = red[row_in_tile] + red[BM + row_in_tile];
            stats[BM + row_in_tile] = red[2 * BM + row_in_tile] + red[3 * BM + row_in_tile];
        }
    }
    __syncwarp();
    ptx::cluster_sync_acq_rel();  // #1: every CTA's row statistics are visible
    if (is_epi) {
        float t1 = 0.0f, t2 = 0.0f;
#pragma unroll
        for (int i = 0; i < NPEERS; ++i) {
            t1 += ptx::ld_shared_cluster_f32(&stats[row_in_tile], peer_first + i * peer_step);
            t2 += ptx::ld_shared_cluster_f32(&stats[BM + row_in_tile], peer_first + i * peer_step);
        }
        mean = t1 * inv_n;
        // mean of squared deviations from the fp32 sums; clamped at zero against rounding
        const float var = fmaxf(fmaf(-mean, mean, t2 * inv_n), 0.0f);
        rstd = 1.0f / sqrtf(var + la.eps);
        // pass B: normalise, scale, shift, store.  Every lane takes part in the (warp-collective) TMEM loads;
        // only the global stores are guarded by the row bound.
        if (epi_ok) {
            // every product has finished (tmem_full), so the first pipeline stage is free to stage the output
            uint8_t* stage_tile = out_stage + (warp - 2) * 4096;
            uint8_t* stage_row = stage_tile + lane * 128;
#pragma unroll 1
            for (int c = 0; c < 4; c += G) {
                uint32_t r[G][32];
                uint4 rg[G][4], rb[G][4];
#pragma unroll
                for (int u = 0; u < G; ++u) ptx::tmem_ld_32x32b_x32(t_base + (c + u) * 32, r[u]);
#pragma unroll
                for (int u = 0; u < G; ++u) {
                    const int col0 = col_base + (c + u) * 32;
                    if (la.gamma) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) rg[u][g] = __ldg(reinterpret_cast<const uint4*>(la.gamma + col0 + g * 8));
                    }
                    if (la.beta) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) rb[u][g] = __ldg(reinterpret_cast<const uint4*>(la.beta + col0 + g * 8));
                    }
                }
                ptx::tmem_ld_wait();
                if (((c & 1) == 0)) {  // first chunk of a 64-column staging tile
                    if (lane == 0) ptx::tma_store_wait_read<0>();  // the previous store has read the staging tile
                    __syncwarp();
                }
#pragma unroll
                for (int u = 0; u < G; ++u) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        float gm[8], bt[8], o[8];
                        if (la.gamma) unpack8(rg[u][g], gm);
                        if (la.beta) unpack8(rb[u][g], bt);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            float v = (__uint_as_float(r[u][g * 8 + j]) - mean) * rstd;
                            if (la.gamma) v *= gm[j];
                            if (la.beta) v += bt[j];
                            o[j] = v;
                        }
                        *reinterpret_cast<uint4*>(stage_row + (((((c + u) & 1) * 4 + g) ^ (lane & 7)) << 4)) = pack8(o);
                    }
                }
                if (((c + G) & 1) == 0) {  // the staging tile is complete
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        ptx::tma_store_4d(tmap_c, stage_tile, col_base + (c + G - 2) * 32, m0 + quarter * 32, 0, 0);
                        ptx::tma_store_commit();
                    }
                }
            }
            if (lane == 0) ptx::tma_store_wait<0>();  // the bulk stores have landed before the CTA may leave
        }
    }
}

}  // namespace gemm
}  // namespace b200ml
