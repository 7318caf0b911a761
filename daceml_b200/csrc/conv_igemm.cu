// k x k convolution with stride 1 or 2 (NCHW, fp32, group 1) as an implicit GEMM on the tensor cores, fp32-grade
// accuracy ("3 x TF32"):
//     Y[n, m, h, w] = act(B[m] + sum_{c, i, j} W[m, c, i, j] * X[n, c, sh h - pad_top + i, sw w - pad_left + j]) + R[n, m, h, w]
// (the reference's routes: the loop nest of daceml/onnx/op_implementations/img_op_implementations.py:217-288 and cuDNN,
// cudnn_implementations.py:123-410).
//
// No im2col buffer exists anywhere.  A tile is 8 output rows x 32 output columns of one image (two accumulators of 128
// pixels: one TMEM lane per pixel) times a block of up to 128 output channels (TMEM columns).  The reduction runs over
// (8 input channels) x (kernel column j) "stages", each of which serves the kh kernel rows:
//   * TMA brings the raw input window of 8 channels (8 + kh - 1 rows, 32 + halo columns; the tensor map fills the
//     padding and the channels past C with zeros) into shared memory once per 8 channels;
//   * eight split warps (one channel each) write, for kernel column j, the window shifted by j as an MN-major tf32
//     operand - hi part and lo part - in the 128-byte swizzle with 32-byte atoms: one 512-byte atom per (image row,
//     group of 4 channels), 32 pixels per 128-byte line.  A shift by j is not a multiple of 16 bytes, which is why it is
//     made here and not by the tensor map;
//   * kernel row i needs no copy: its operand is the same shifted window starting i atoms (image rows) further down,
//     so the three or five products of a stage differ only in their descriptors' start addresses;
//   * the weights of the stage (8 channels x kh rows x the channel block, hi and lo, split once per call by a small
//     kernel into an [.., c, j, i, m] order) arrive by TMA as the N-major operand in the same swizzle.
// The tensor core accumulates X_lo.W_hi + X_hi.W_lo + X_hi.W_hi per kernel row and half tile.  Bias, activation and
// residual are applied by sixteen epilogue warps (a lane = a pixel of one output row), which stage [8 channels][32 pixels]
// boxes in shared memory and send them with bulk tensor stores; those clip the columns past the image and the channels
// past M.  Roles as in the 1x1 kernel: warp 0 TMA, warp 1 MMA and TMEM owner, warps 2-9 split, warps 10-25 epilogue;
// one persistent CTA per SM; two accumulator sets, so a tile's epilogue runs under the next tile's products.
//
// Two variations.  DIRECT: images whose rows the TMA unit cannot describe (width not a multiple of 4 elements) - each split
// warp copies its channel's window with asynchronous 4-byte copies (cp.async, zero fill for the padding), one channel
// block ahead, and the epilogue warps store Y themselves.
// Narrow images (output width <= 16, always DIRECT): an operand line holds two image rows, 8 apart, of 16 columns, so a
// tile is 16 rows x 16 columns; kernel row i is still "i lines further down" for both rows of a line.
// Stride (sh, sw): the split warps pick every sw-th column of the window when they write a line, and output row r of a
// half tile, kernel row i, is line sh r + i - the operand's atoms are sh lines apart instead of one.
#include "conv_tc.cuh"

namespace b200ml {

using namespace convtc;

namespace {

constexpr int IG_KC = 8;                       // input channels per stage = one tf32 MMA step
constexpr int IG_ROWS = 8, IG_COLS = 32;       // output tile: two halves of 4 rows x 32 columns = 2 x 128 pixels
constexpr int IG_RAW_SLOTS = 2;
constexpr int IG_MAX_STAGES = 6;
constexpr int IG_SPLIT_WARPS = IG_KC, IG_EPI_WARPS = 16;  // one split warp per channel of a stage
constexpr int IG_FIRST_EPI = 2 + IG_SPLIT_WARPS;
constexpr int IG_THREADS = 32 * (2 + IG_SPLIT_WARPS + IG_EPI_WARPS);
constexpr int IG_OUT_BYTES = 2 * 8 * 32 * 4;   // per epilogue warp: two [8 channels][32 pixels] boxes
constexpr int IG_BAR_BYTES = 256;
constexpr int IG_SMEM_LIMIT = 227 * 1024;

struct IgArgs {
    int32_t c, m, oh, ow, kh, kw;
    int32_t cblocks, nb, nblocks, hblocks, wblocks, num_tiles;
    int32_t parts, cw;                    // a 128-byte operand line = `parts` image rows (8 apart) of `cw` = 32 / parts columns
    int32_t rb, rr, wb, xoff;             // window: operand lines, raw rows, raw columns, column of kernel column 0 for output column 0
    int32_t pla, pad_top;                 // the window starts pla columns left of the tile and pad_top rows above it
    int32_t sh, sw;                       // strides (1 or 2): output row r reads lines sh r + i, output column w raw column sw w + j
    int32_t stages, raw_bytes, stage_bytes, shift_bytes;
    int32_t act;
    int32_t direct_io, h, w;  // direct_io: X and Y cannot be described to the TMA unit (row pitch or base not a multiple of
                              // 16 bytes); the split warps fetch the window and the epilogue warps store Y themselves
    const float* x;
    float* y;
    const float* bias;      // [M] or null
    const float* residual;  // like Y or null
    int32_t* status;
};

// W [m, c, kh, kw] -> out [2][row][ntot], row = ((c / 8 * kw + j) * kh + i) * 8 + c % 8: hi and lo parts, zero-padded to
// whole 8-channel blocks and to ntot output channels.  Rounded to nearest here (|lo| <= 2^-11 |w|).
__global__ void __launch_bounds__(256) ig_split_weights_kernel(const float* __restrict__ w, float* __restrict__ out, int m,
                                                               int c, int kh, int kw, int ntot, int rows) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t total = static_cast<int64_t>(rows) * ntot;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int row = static_cast<int>(i / ntot), n = static_cast<int>(i - static_cast<int64_t>(row) * ntot);
        const int ch = row & 7, t = row >> 3;
        const int ki = t % kh, kj = (t / kh) % kw, cb = t / (kh * kw);
        const int cc = cb * 8 + ch;
        float v = 0.0f;
        if (n < m && cc < c) v = __ldg(w + ((static_cast<int64_t>(n) * c + cc) * kh + ki) * kw + kj);
        const uint32_t b = __float_as_uint(v);
        const bool finite = (b & 0x7f800000u) != 0x7f800000u;
        const float hi = __uint_as_float(finite ? ((b + 0xfffu + ((b >> 13) & 1u)) & 0xffffe000u) : b);
        out[i] = hi;
        out[total + i] = finite ? v - hi : 0.0f;
    }
}

struct IgTile {
    int n, nblk, h0, w0;
};
__device__ __forceinline__ IgTile ig_tile(const IgArgs& a, int tile) {
    IgTile t;
    const int wblk = tile % a.wblocks;
    tile /= a.wblocks;
    const int hblk = tile % a.hblocks;
    tile /= a.hblocks;
    t.nblk = tile % a.nblocks;
    t.n = tile / a.nblocks;
    t.h0 = hblk * IG_ROWS * a.parts;
    t.w0 = wblk * a.cw;
    return t;
}

// Direct mode: a split warp copies its channel's window of a channel block into its part of a raw slot with asynchronous
// 4-byte copies (lane = window column, and column + 32); padding and channels past C are written as zeros (source size
// 0).  The copies of the next block fly while the warp works on the current one; nothing is held in registers.
__device__ __forceinline__ void ig_prefetch_window(uint32_t dst, const IgArgs& a, const IgTile& t, int cb, int ch, int lane) {
    const int c = cb * IG_KC + ch;
    const float* xc = a.x + (static_cast<int64_t>(t.n) * a.c + (c < a.c ? c : 0)) * a.h * a.w;
    const int gy0 = t.h0 * a.sh - a.pad_top, gx0 = t.w0 * a.sw - a.pla;
    for (int r = 0; r < a.rr; ++r) {
        const int gy = gy0 + r;
        const bool r_ok = c < a.c && gy >= 0 && gy < a.h;
#pragma unroll
        for (int hc = 0; hc < 3; ++hc) {  // the window is at most 96 columns wide (stride 2: 62 + kernel + alignment)
            const int col = lane + 32 * hc, gx = gx0 + col;
            if (col < a.wb) {
                const bool ok = r_ok && gx >= 0 && gx < a.w;
                const float* src = ok ? xc + static_cast<int64_t>(gy) * a.w + gx : a.x;
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst + (r * a.wb + 32 * hc) * 4), "l"(src), "r"(ok ? 4 : 0) : "memory");
            }
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}
__device__ __forceinline__ void ig_prefetch_wait() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Direct mode: two finished 8-channel units of 32 pixels straight to Y (lane = pixel: a warp writes whole row pieces).
template <int ACT, bool RES>
__device__ __forceinline__ void ig_finish_direct(const uint32_t (&r)[2][8], const float (&rv)[2][8], float* ya, float* yb, int64_t plane,
                                                 int na, int nb) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float va = pw_act<ACT>(__uint_as_float(r[0][j]));
        float vb = pw_act<ACT>(__uint_as_float(r[1][j]));
        if (RES) va += rv[0][j], vb += rv[1][j];
        if (j < na) ya[j * plane] = va;
        if (j < nb) yb[j * plane] = vb;
    }
}

// One split warp's share of a stage: its channel's window rows, shifted by the kernel column (already in `src`), as hi
// and lo lines of the operand.  Four rows at a time: the loads are independent, the stores follow.
__device__ __forceinline__ void ig_split_stage(uint32_t src, uint32_t hi, uint32_t lo, int rb, int wb) {
#pragma unroll 1
    for (int r0 = 0; r0 < rb; r0 += 4) {
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = r0 + u < rb ? ld_shared_f32(src + (r0 + u) * wb * 4) : 0.0f;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (r0 + u < rb) {
                float h, l;
                split_tf32(v[u], h, l);
                st_shared_f32(hi + (r0 + u) * 1024, h);
                st_shared_f32(lo + (r0 + u) * 1024, l);
            }
        }
    }
}

// DIRECT: X and Y do not go through the TMA unit (see IgArgs::direct_io).
template <bool DIRECT>
__global__ void __launch_bounds__(IG_THREADS, 1)
conv_igemm_tf32x3_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                         const __grid_constant__ CUtensorMap tmap_y, const IgArgs args) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // [stages][shifted X hi, lo | W hi, lo]  [raw slots]  [epilogue staging]  [barriers]
    uint8_t* raw_base = smem + args.stages * args.stage_bytes;
    uint8_t* out_stage = raw_base + IG_RAW_SLOTS * args.raw_bytes;
    uint64_t* ready = reinterpret_cast<uint64_t*>(out_stage + IG_EPI_WARPS * IG_OUT_BYTES);  // W bytes + the split warps
    uint64_t* empty = ready + IG_MAX_STAGES;
    uint64_t* raw_full = empty + IG_MAX_STAGES;
    uint64_t* raw_empty = raw_full + IG_RAW_SLOTS;
    uint64_t* tmem_full = raw_empty + IG_RAW_SLOTS;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    uint32_t tmem_cols = 32;
    while (tmem_cols < 4u * args.nb) tmem_cols <<= 1;
    const uint32_t acc_stride = tmem_cols / 2, half_stride = tmem_cols / 4;  // [accumulator set][half tile][channel]
    const int natoms = args.nb / 32;                                          // 32-channel atoms of the weight operand
    const int w_part_bytes = natoms * args.kh * 1024;                         // W_hi (or W_lo) of a stage
    const int x_part_bytes = args.rb * 1024;                                  // X_hi (or X_lo) of a stage

    if (warp == 0 && lane == 0) {
        ptx::prefetch_tensormap(&tmap_x);
        ptx::prefetch_tensormap(&tmap_w);
        ptx::prefetch_tensormap(&tmap_y);
    }
    if (warp == 1) {
        if (lane == 0) {
            for (int s = 0; s < args.stages; ++s) {
                ptx::mbar_init(&ready[s], 1 + IG_SPLIT_WARPS);
                ptx::mbar_init(&empty[s], 1);
            }
            for (int r = 0; r < IG_RAW_SLOTS; ++r) {
                ptx::mbar_init(&raw_full[r], 1);
                ptx::mbar_init(&raw_empty[r], IG_SPLIT_WARPS);
            }
            for (int a = 0; a < 2; ++a) {
                ptx::mbar_init(&tmem_full[a], 1);
                ptx::mbar_init(&tmem_empty[a], IG_EPI_WARPS);
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
    pdl_wait();  // the split weights (and possibly X, the residual) come from kernels before this one in the stream

    if (warp == 0) {
        // ------------------------------ TMA producer: raw windows and weight chunks ------------------------------
        if (ptx::elect_one()) {
            int stage = 0, slot = 0;
            uint32_t phase = 0, slot_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < args.num_tiles; tile += gridDim.x) {
                const IgTile t = ig_tile(args, tile);
                for (int cb = 0; ok && cb < args.cblocks; ++cb) {
                    if constexpr (!DIRECT) {
                        if (!ptx::mbar_wait_suspend(&raw_empty[slot], slot_phase ^ 1)) {
                            atomicExch(args.status, DEV_TIMEOUT_PRODUCER);
                            ok = false;
                            break;
                        }
                        ptx::mbar_expect_tx(&raw_full[slot], static_cast<uint32_t>(args.wb * args.rr * IG_KC * 4));
                        // x is a multiple of 4 elements (16 bytes); rows and columns outside the image arrive as zeros
                        ptx::tma_load_4d(raw_base + slot * args.raw_bytes, &tmap_x, &raw_full[slot], t.w0 * args.sw - args.pla,
                                         t.h0 * args.sh - args.pad_top, cb * IG_KC, t.n);
                        if (++slot == IG_RAW_SLOTS) {
                            slot = 0;
                            slot_phase ^= 1;
                        }
                    }
                    for (int kj = 0; kj < args.kw; ++kj) {
                        if (!ptx::mbar_wait_suspend(&empty[stage], phase ^ 1)) {
                            atomicExch(args.status, DEV_TIMEOUT_PRODUCER);
                            ok = false;
                            break;
                        }
                        uint8_t* wst = smem + stage * args.stage_bytes + args.shift_bytes;
                        ptx::mbar_expect_tx(&ready[stage], static_cast<uint32_t>(2 * w_part_bytes));
                        const int row0 = (cb * args.kw + kj) * args.kh * IG_KC;
                        for (int part = 0; part < 2; ++part)
                            for (int a = 0; a < natoms; ++a)
                                ptx::tma_load_4d(wst + part * w_part_bytes + a * args.kh * 1024, &tmap_w, &ready[stage],
                                                 t.nblk * args.nb + a * 32, row0, part, 0);
                        if (++stage == args.stages) {
                            stage = 0;
                            phase ^= 1;
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (ptx::elect_one()) {
            const uint32_t idesc = pw_idesc(static_cast<uint32_t>(args.nb), 1u);
            const uint64_t d_x_first = make_smem_desc_sw128_base32(ptx::smem_u32(smem), args.sh * 1024, 512);  // output rows are sh lines apart
            const uint64_t d_w_first = make_smem_desc_sw128_base32(ptx::smem_u32(smem) + args.shift_bytes, args.kh * 1024, 512);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int it = 0;
            for (int tile = blockIdx.x; ok && tile < args.num_tiles; tile += gridDim.x, ++it) {
                const int acc = it & 1;
                if (!ptx::mbar_wait_suspend(&tmem_empty[acc], ((it >> 1) & 1) ^ 1)) {
                    atomicExch(args.status, DEV_TIMEOUT_MMA);
                    break;
                }
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * acc_stride;
                const int nstages = args.cblocks * args.kw;
                for (int st = 0; st < nstages; ++st) {
                    if (!ptx::mbar_wait(&ready[stage], phase)) {
                        atomicExch(args.status, DEV_TIMEOUT_MMA);
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    // descriptors differ only in their start address field (bytes / 16): one 64-bit add each
                    const uint64_t d_xh0 = d_x_first + static_cast<uint32_t>(stage * (args.stage_bytes >> 4));
                    const uint64_t d_wh0 = d_w_first + static_cast<uint32_t>(stage * (args.stage_bytes >> 4));
                    for (int ki = 0; ki < args.kh; ++ki) {
                        // W: N-major, 32-channel atoms kh KB apart, 4-channel (K) groups 512 bytes apart; kernel row ki is 1 KB in
                        const uint64_t d_wh = d_wh0 + static_cast<uint32_t>(ki * 64), d_wl = d_wh + static_cast<uint32_t>(w_part_bytes >> 4);
#pragma unroll
                        for (int hf = 0; hf < 2; ++hf) {
                            // X: MN-major, one atom per image row (1 KB apart: two 4-channel groups of 512 bytes); kernel
                            // row ki of half hf starts at window row 4 hf + ki
                            const uint64_t d_xh = d_xh0 + static_cast<uint32_t>((4 * hf * args.sh + ki) * 64), d_xl = d_xh + static_cast<uint32_t>(x_part_bytes >> 4);
                            const uint32_t d = d_tmem + hf * half_stride;
                            pw_mma(d, d_xl, d_wh, idesc, (st | ki) != 0 ? 1u : 0u);  // the two small terms first
                            pw_mma(d, d_xh, d_wl, idesc, 1u);
                            pw_mma(d, d_xh, d_wh, idesc, 1u);
                        }
                    }
                    ptx::mma_commit(&empty[stage]);
                    if (++stage == args.stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                ptx::mma_commit(&tmem_full[acc]);
            }
        }
    } else if (warp < IG_FIRST_EPI) {
        // ------------------------------ split: raw window -> shifted hi / lo operands ------------------------------
        // Warp = one of the 8 channels of the stage, lane = output column.  For kernel column kj the value under output
        // column `lane` of window row r is raw[ch][r][xoff + kj + lane]; it goes to line (ch & 3) of atom (r, ch >> 2) of
        // the stage, 32-byte chunk (lane / 8) ^ (ch & 3): a warp reads and writes whole 128-byte lines, conflict-free.
        const int ch = warp - 2, cr = ch & 3;
        const uint32_t dst_lane = (ch >> 2) * 512 + cr * 128 + ((lane * 4) ^ (cr << 5));
        int stage = 0, slot = 0;
        uint32_t phase = 0, slot_phase = 0;
        bool ok = true;
        const uint32_t my_raw = ptx::smem_u32(raw_base) + (ch * args.rr * args.wb + lane) * 4;  // this warp's channel, slot 0
        if constexpr (DIRECT) if (blockIdx.x < args.num_tiles) ig_prefetch_window(my_raw, args, ig_tile(args, blockIdx.x), 0, ch, lane);
        for (int tile = blockIdx.x; ok && tile < args.num_tiles; tile += gridDim.x) {
            for (int cb = 0; ok && cb < args.cblocks; ++cb) {
                if constexpr (DIRECT) {
                    // this warp alone writes and reads its channel of the window: no barrier, its own copies' completion
                    // and program order are enough; the other slot is free (the block that used it is done)
                    ig_prefetch_wait();
                    __syncwarp();
                    const bool last_cb = cb + 1 == args.cblocks;
                    const int next_tile = last_cb ? tile + gridDim.x : tile;
                    if (next_tile < args.num_tiles)
                        ig_prefetch_window(my_raw + (slot ^ 1) * args.raw_bytes, args, ig_tile(args, next_tile), last_cb ? 0 : cb + 1, ch, lane);
                } else {
                    ok = __all_sync(0xffffffffu, ptx::mbar_wait_suspend(&raw_full[slot], slot_phase));
                    if (!ok) {
                        if (lane == 0) atomicExch(args.status, DEV_TIMEOUT_EPILOGUE);
                        break;
                    }
                }
                // lane = (part, column): part j of operand line L is raw row L + 8 sh j; column w reads raw column sw w + kj
                const uint32_t src0 = ptx::smem_u32(raw_base + slot * args.raw_bytes) +
                                      ((ch * args.rr + 8 * args.sh * (lane / args.cw)) * args.wb + args.xoff + args.sw * (lane % args.cw)) * 4;
                for (int kj = 0; kj < args.kw; ++kj) {
                    ok = __all_sync(0xffffffffu, ptx::mbar_wait_suspend(&empty[stage], phase ^ 1));
                    if (!ok) {
                        if (lane == 0) atomicExch(args.status, DEV_TIMEOUT_EPILOGUE);
                        break;
                    }
                    const uint32_t hi = ptx::smem_u32(smem + stage * args.stage_bytes) + dst_lane, lo = hi + x_part_bytes;
                    const uint32_t src = src0 + kj * 4;
                    ig_split_stage(src, hi, lo, args.rb, args.wb);
                    ptx::fence_proxy_async_smem();  // the tensor core reads shared memory through the async proxy
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&ready[stage]);
                    if (++stage == args.stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                __syncwarp();
                if (lane == 0 && !DIRECT) ptx::mbar_arrive(&raw_empty[slot]);  // this warp has read its channel of the window
                if (++slot == IG_RAW_SLOTS) {
                    slot = 0;
                    slot_phase ^= 1;
                }
            }
        }
    } else {
        // ------------------------------ epilogue: one output row x every fourth 8-channel unit per warp ------------------------------
        const int quarter = warp & 3;                      // TMEM lanes [32 q, 32 q + 32): a warp may only touch its own quarter
        const int group = (warp - IG_FIRST_EPI) >> 2;      // units group, group + 4, ...
        constexpr int NGROUPS = IG_EPI_WARPS / 4;
        uint8_t* stg = out_stage + (warp - IG_FIRST_EPI) * IG_OUT_BYTES;
        const uint32_t stg_lane = ptx::smem_u32(stg) + lane * 4;
        const int64_t plane = static_cast<int64_t>(args.oh) * args.ow;
        int it = 0;
        for (int tile = blockIdx.x; tile < args.num_tiles; tile += gridDim.x, ++it) {
            const int acc = it & 1;
            const IgTile t = ig_tile(args, tile);
            if (!__all_sync(0xffffffffu, ptx::mbar_wait_suspend(&tmem_full[acc], (it >> 1) & 1))) {
                if (lane == 0) atomicExch(args.status, DEV_TIMEOUT_EPILOGUE);
                break;
            }
            ptx::tc_fence_after();
            const int m0 = t.nblk * args.nb;                                   // first output channel of the block
            const int nunits = ((args.m - m0 < args.nb ? args.m - m0 : args.nb) + 7) / 8;
            const int col = t.w0 + lane % args.cw;   // lane = (part, column); one part of 32 columns with TMA stores
#pragma unroll 1
            for (int hf = 0; hf < 2; ++hf) {
                const int row = t.h0 + 4 * hf + quarter + 8 * (lane / args.cw);
                const bool p_ok = col < args.ow && row < args.oh;
                if (!__any_sync(0xffffffffu, p_ok)) continue;  // rows past the image have nothing to store
                const uint32_t t_base = tmem_base + acc * acc_stride + hf * half_stride + (static_cast<uint32_t>(quarter * 32) << 16);
                const float* res = args.residual
                                       ? args.residual + (static_cast<int64_t>(t.n) * args.m + m0) * plane + static_cast<int64_t>(row) * args.ow + col
                                       : nullptr;
#pragma unroll 1
                for (int ua = group; ua < nunits; ua += 2 * NGROUPS) {
                    const int ub = ua + NGROUPS;
                    const bool two = ub < nunits;  // warp-uniform
                    const int ca = ua * 8, cb = two ? ub * 8 : ca;
                    uint32_t r[2][8];
                    float rv[2][8], bv[2][8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        bv[0][j] = (args.bias && m0 + ca + j < args.m) ? __ldg(args.bias + m0 + ca + j) : 0.0f;
                        bv[1][j] = (args.bias && m0 + cb + j < args.m) ? __ldg(args.bias + m0 + cb + j) : 0.0f;
                    }
                    if (res) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            rv[0][j] = (p_ok && m0 + ca + j < args.m) ? __ldg(res + static_cast<int64_t>(ca + j) * plane) : 0.0f;
                            rv[1][j] = (p_ok && m0 + cb + j < args.m) ? __ldg(res + static_cast<int64_t>(cb + j) * plane) : 0.0f;
                        }
                    }
                    ptx::tmem_ld_32x32b_x8(t_base + ca, r[0]);
                    ptx::tmem_ld_32x32b_x8(t_base + cb, r[1]);
                    if (lane == 0) ptx::tma_store_wait_read<0>();  // the stores of the last turn have read the staging boxes
                    ptx::tmem_ld_wait();
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        r[0][j] = __float_as_uint(__uint_as_float(r[0][j]) + bv[0][j]);
                        r[1][j] = __float_as_uint(__uint_as_float(r[1][j]) + bv[1][j]);
                    }
                    if constexpr (DIRECT) {
                        float* yo = args.y + (static_cast<int64_t>(t.n) * args.m + m0) * plane + static_cast<int64_t>(row) * args.ow + col;
                        const int na = p_ok ? args.m - (m0 + ca) : 0, nb2 = (p_ok && two) ? args.m - (m0 + cb) : 0;  // channels to store (8 or fewer)
                        float *ya = yo + ca * plane, *yb = yo + cb * plane;
                        if (res) {
                            if (args.act == B200ML_EPI_SWISH) ig_finish_direct<B200ML_EPI_SWISH, true>(r, rv, ya, yb, plane, na, nb2);
                            else if (args.act == 0) ig_finish_direct<0, true>(r, rv, ya, yb, plane, na, nb2);
                            else if (args.act == B200ML_EPI_RELU) ig_finish_direct<B200ML_EPI_RELU, true>(r, rv, ya, yb, plane, na, nb2);
                            else ig_finish_direct<B200ML_EPI_GELU, true>(r, rv, ya, yb, plane, na, nb2);
                        } else {
                            if (args.act == B200ML_EPI_SWISH) ig_finish_direct<B200ML_EPI_SWISH, false>(r, rv, ya, yb, plane, na, nb2);
                            else if (args.act == 0) ig_finish_direct<0, false>(r, rv, ya, yb, plane, na, nb2);
                            else if (args.act == B200ML_EPI_RELU) ig_finish_direct<B200ML_EPI_RELU, false>(r, rv, ya, yb, plane, na, nb2);
                            else ig_finish_direct<B200ML_EPI_GELU, false>(r, rv, ya, yb, plane, na, nb2);
                        }
                        continue;
                    }
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
                        ptx::tma_store_4d(&tmap_y, stg, t.w0, row, m0 + ca, t.n);  // columns past OW and channels past M are clipped
                        if (two) ptx::tma_store_4d(&tmap_y, stg + 1024, t.w0, row, m0 + cb, t.n);
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

// The shape of the launch: channel block, window, stages, shared memory.  `ok` is false when nothing fits.
struct IgPlan {
    bool ok;
    int nb, nblocks, ntot, cblocks, rows, rb, wb, pla, stages, raw_bytes, shift_bytes, stage_bytes, smem;
    int parts, cw, rr;
};

IgPlan ig_plan(const b200ml_conv_params* p, int64_t ow) {
    IgPlan pl{};
    // narrow images: two image rows (8 apart) of 16 columns per operand line, i.e. tiles of 16 x 16 instead of 8 x 32
    pl.parts = ow <= 16 ? 2 : 1;
    pl.cw = 32 / pl.parts;
    const int sh = (int)p->stride_h, sw = (int)p->stride_w;
    pl.rr = (IG_ROWS * pl.parts - 1) * sh + (int)p->kh;
    const int kh = (int)p->kh, kw = (int)p->kw;
    pl.cblocks = (int)ceil_div(p->c, IG_KC);
    pl.rows = pl.cblocks * kw * kh * IG_KC;
    pl.rb = (IG_ROWS - 1) * sh + kh;  // operand lines: output row r of a half, kernel row i -> line sh r + i
    pl.pla = (int)ceil_div(p->pad_left, 4) * 4;
    pl.wb = (int)ceil_div(pl.pla - p->pad_left + kw + (pl.cw - 1) * sw, 4) * 4;
    pl.raw_bytes = (int)ceil_div((int64_t)pl.wb * pl.rr * IG_KC * 4, 1024) * 1024;
    pl.shift_bytes = 2 * pl.rb * 1024;
    const int fixed = IG_RAW_SLOTS * pl.raw_bytes + IG_EPI_WARPS * IG_OUT_BYTES + IG_BAR_BYTES + 1024 /* alignment */;
    // the widest channel block that leaves three stages (two if there is no other way)
    for (int want = 3; want >= 2 && !pl.ok; --want) {
        for (int nb = 128; nb >= 32 && !pl.ok; nb /= 2) {
            const int use = p->m <= nb ? (int)ceil_div(p->m, 32) * 32 : nb;
            const int stage = pl.shift_bytes + 2 * (use / 32) * kh * 1024;
            const int stages = (IG_SMEM_LIMIT - fixed) / stage;
            if (stages >= want) {
                pl.ok = true;
                pl.nb = use;
                pl.stage_bytes = stage;
                pl.stages = stages < IG_MAX_STAGES ? stages : IG_MAX_STAGES;
            }
        }
    }
    if (!pl.ok) return pl;
    pl.nblocks = (int)ceil_div(p->m, pl.nb);
    pl.ntot = pl.nblocks * pl.nb;
    pl.smem = pl.stages * pl.stage_bytes + fixed;
    return pl;
}

bool conv_tc_enabled() {
    static const bool on = [] {
        const char* e = getenv("B200ML_CONV_TC");
        return !(e && e[0] == '0');
    }();
    return on;
}

}  // namespace

// Whether the implicit-GEMM kernel covers this convolution (the caller uses the direct FP32-FMA kernel otherwise).
bool conv_igemm_applies(const b200ml_ctx* ctx, const b200ml_conv_params* p, int64_t oh, int64_t ow) {
    if (!conv_tc_enabled() || p->dtype != B200ML_F32 || !ctx->encode_tiled) return false;
    if (p->group != 1 || p->gate) return false;
    if (p->kh > 7 || p->kw > 7) return false;
    if (p->kh * p->kw < 2 && p->stride_h == 1 && p->stride_w == 1) return false;  // the 1x1 kernel's case
    if (p->stride_h > 2 || p->stride_w > 2 || p->dil_h != 1 || p->dil_w != 1) return false;
    if (p->pad_top > 8 || p->pad_left > 8 || p->pad_bottom > 8 || p->pad_right > 8) return false;
    if (p->c * p->kh * p->kw < 64 || p->m < 16) return false;                 // short reductions stay on the FP32 pipe
    if (p->n * oh * ow < 4 * 1024) return false;                              // too little work for two launches
    const IgPlan pl = ig_plan(p, ow);
    if (!pl.ok) return false;
    if (2ll * pl.rows * pl.ntot * 4 > ctx->workspace_bytes) return false;     // the split weights live in the context's scratch
    const int64_t tiles = p->n * pl.nblocks * ceil_div(oh, IG_ROWS * pl.parts) * ceil_div(ow, pl.cw);
    if (tiles >= (1ll << 31) || p->h >= (1 << 24) || p->w >= (1 << 24) || p->c >= (1 << 24) || p->m >= (1 << 24) || p->n >= (1 << 24)) return false;
    if (p->n * p->c * p->h * p->w * 4 >= (1ll << 40) || p->n * p->m * oh * ow * 4 >= (1ll << 40)) return false;  // tensor-map strides are below 2^40 bytes
    return true;
}

int64_t conv_igemm_pack_bytes(const b200ml_conv_params* p, int64_t ow) {
    const IgPlan pl = ig_plan(p, ow);
    return pl.ok ? 2ll * pl.rows * pl.ntot * 4 : 0;
}

int conv_igemm_pack(const b200ml_ctx*, const b200ml_conv_params* p, int64_t ow, void* dst, cudaStream_t stream) {
    const IgPlan pl = ig_plan(p, ow);
    const int64_t total = (int64_t)pl.rows * pl.ntot;
    const unsigned grid = (unsigned)(ceil_div(total, 256) < 1184 ? ceil_div(total, 256) : 1184);
    B200ML_CUDA(launch_pdl(ig_split_weights_kernel, dim3(grid), dim3(256), 0, stream, static_cast<const float*>(p->weight),
                           static_cast<float*>(dst), (int)p->m, (int)p->c, (int)p->kh, (int)p->kw, pl.ntot, pl.rows));
    return check_launch("ig_split_weights");
}

int conv_igemm(const b200ml_ctx* ctx, const b200ml_conv_params* p, int64_t oh, int64_t ow, cudaStream_t stream) {
    const IgPlan pl = ig_plan(p, ow);
    float* wsplit = static_cast<float*>(ctx->workspace);
    if (p->packed_weight) {  // split once by the caller
        B200ML_REQUIRE(aligned16(p->packed_weight), "conv: the packed weights must be 16-byte aligned");
        wsplit = const_cast<float*>(static_cast<const float*>(p->packed_weight));
    } else {
        int rc = conv_igemm_pack(ctx, p, ow, wsplit, stream);
        if (rc) return rc;
    }
    CUtensorMap tx, tw, ty;
    // X and Y go through the TMA unit when their row pitches and bases are multiples of 16 bytes
    // (and tiles of one row of 32 columns per operand line: the bulk stores write [8 channels][32 columns] boxes)
    const bool direct_io = pl.parts != 1 || p->w % 4 != 0 || ow % 4 != 0 || !aligned16(p->x) || !aligned16(p->y);
    if (!direct_io) {
        const cuuint64_t dims[4] = {(cuuint64_t)p->w, (cuuint64_t)p->h, (cuuint64_t)p->c, (cuuint64_t)p->n};
        const cuuint64_t strides[3] = {(cuuint64_t)p->w * 4, (cuuint64_t)p->w * p->h * 4, (cuuint64_t)p->w * p->h * p->c * 4};
        const cuuint32_t box[4] = {(cuuint32_t)pl.wb, (cuuint32_t)pl.rr, IG_KC, 1};
        CUresult r = encode_tiled_cached(ctx, &tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, p->x, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (r != CUDA_SUCCESS) return fail(B200ML_ERR_CUDA, "conv k x k: cuTensorMapEncodeTiled(X) failed with CUresult %d", (int)r);
    }
    {
        const cuuint64_t dims[4] = {(cuuint64_t)pl.ntot, (cuuint64_t)pl.rows, 2, 1};
        const cuuint64_t strides[3] = {(cuuint64_t)pl.ntot * 4, (cuuint64_t)pl.ntot * 4 * pl.rows, (cuuint64_t)pl.ntot * 4 * pl.rows * 2};
        const cuuint32_t box[4] = {32, (cuuint32_t)(p->kh * IG_KC), 1, 1};
        CUresult r = encode_tiled_cached(ctx, &tw, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, wsplit, dims, strides, box,
                                         CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
        if (r != CUDA_SUCCESS) return fail(B200ML_ERR_CUDA, "conv k x k: cuTensorMapEncodeTiled(W) failed with CUresult %d", (int)r);
    }
    if (direct_io) {
        tx = tw;  // never used for a copy; the kernel's parameters still have to be valid maps
        ty = tw;
    } else {
        const cuuint64_t dims[4] = {(cuuint64_t)ow, (cuuint64_t)oh, (cuuint64_t)p->m, (cuuint64_t)p->n};
        const cuuint64_t strides[3] = {(cuuint64_t)ow * 4, (cuuint64_t)ow * oh * 4, (cuuint64_t)ow * oh * p->m * 4};
        const cuuint32_t box[4] = {32, 1, 8, 1};
        CUresult r = encode_tiled_cached(ctx, &ty, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, p->y, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (r != CUDA_SUCCESS) return fail(B200ML_ERR_CUDA, "conv k x k: cuTensorMapEncodeTiled(Y) failed with CUresult %d", (int)r);
    }
    IgArgs a{};
    a.c = (int32_t)p->c;
    a.m = (int32_t)p->m;
    a.oh = (int32_t)oh;
    a.ow = (int32_t)ow;
    a.kh = (int32_t)p->kh;
    a.kw = (int32_t)p->kw;
    a.cblocks = pl.cblocks;
    a.nb = pl.nb;
    a.nblocks = pl.nblocks;
    a.parts = pl.parts;
    a.cw = pl.cw;
    a.rr = pl.rr;
    a.hblocks = (int32_t)ceil_div(oh, IG_ROWS * pl.parts);
    a.wblocks = (int32_t)ceil_div(ow, pl.cw);
    a.num_tiles = (int32_t)(p->n * pl.nblocks * a.hblocks * a.wblocks);
    a.rb = pl.rb;
    a.wb = pl.wb;
    a.pla = pl.pla;
    a.xoff = pl.pla - (int32_t)p->pad_left;
    a.pad_top = (int32_t)p->pad_top;
    a.sh = (int32_t)p->stride_h;
    a.sw = (int32_t)p->stride_w;
    a.stages = pl.stages;
    a.raw_bytes = pl.raw_bytes;
    a.stage_bytes = pl.stage_bytes;
    a.shift_bytes = pl.shift_bytes;
    a.act = p->act & (B200ML_EPI_RELU | B200ML_EPI_SWISH | B200ML_EPI_GELU);
    a.direct_io = direct_io ? 1 : 0;
    a.h = (int32_t)p->h;
    a.w = (int32_t)p->w;
    a.x = static_cast<const float*>(p->x);
    a.y = static_cast<float*>(p->y);
    a.bias = static_cast<const float*>(p->bias);
    a.residual = static_cast<const float*>(p->residual);
    a.status = ctx->status_dev;
    static int configured[64] = {};
    if (configured[ctx->device & 63] < pl.smem) {
        B200ML_CUDA(cudaFuncSetAttribute(conv_igemm_tf32x3_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, pl.smem));
        B200ML_CUDA(cudaFuncSetAttribute(conv_igemm_tf32x3_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, pl.smem));
        configured[ctx->device & 63] = pl.smem;
    }
    const int grid = a.num_tiles < ctx->sm_count ? a.num_tiles : ctx->sm_count;
    if (direct_io) B200ML_CUDA(launch_pdl(conv_igemm_tf32x3_kernel<true>, dim3(grid), dim3(IG_THREADS), (size_t)pl.smem, stream, tx, tw, ty, a));
    else B200ML_CUDA(launch_pdl(conv_igemm_tf32x3_kernel<false>, dim3(grid), dim3(IG_THREADS), (size_t)pl.smem, stream, tx, tw, ty, a));
    return check_launch("conv_igemm_tf32x3");
}

}  // namespace b200ml
