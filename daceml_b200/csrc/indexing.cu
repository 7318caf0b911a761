// Data-movement operators: strided copies (Slice / Split / Concat / Expand), Gather, Where and 2-D max pooling.
// All are bounded by HBM traffic: one thread moves one 16-byte unit wherever the innermost extent allows it, and
// neighbouring threads touch neighbouring addresses of the output.
#include "common.cuh"

#include <cuda.h>
#include <math_constants.h>

namespace b200ml {

namespace {

constexpr int MAXR = 6;

struct CopyGeom {
    int32_t rank;
    uint32_t shape[MAXR];  // coalesced extents, innermost last
    int64_t xs[MAXR];      // element strides of the source (0 on broadcast axes)
    int64_t ys[MAXR];      // element strides of the destination
};

// y[sum i_d * ys_d] = x[sum i_d * xs_d] over the index space of g.shape; E is the unit that moves
template <typename E>
__global__ void __launch_bounds__(256) strided_copy_kernel(const E* __restrict__ x, E* __restrict__ y, uint64_t total,
                                                           const CopyGeom g) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    // two units per thread and step: both loads are issued before the first store
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += 2 * stride) {
        int64_t xo[2], yo[2];
        const bool second = i + stride < total;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            uint64_t rem = i + u * stride;
            xo[u] = 0, yo[u] = 0;
#pragma unroll
            for (int d = MAXR - 1; d >= 0; --d) {
                if (d < g.rank) {
                    uint64_t c;
                    if (rem < (1ull << 32)) {  // 32-bit division once the remainder fits (always, after the first step or two)
                        const uint32_t r32 = static_cast<uint32_t>(rem);
                        c = r32 % g.shape[d];
                        rem = r32 / g.shape[d];
                    } else {
                        c = rem % g.shape[d];
                        rem = rem / g.shape[d];
                    }
                    xo[u] += static_cast<int64_t>(c) * g.xs[d];
                    yo[u] += static_cast<int64_t>(c) * g.ys[d];
                }
            }
        }
        const E v0 = x[xo[0]];
        E v1 = E();
        if (second) v1 = x[xo[1]];
        y[yo[0]] = v0;
        if (second) y[yo[1]] = v1;
    }
}

// Up to eight copies in one launch (the parts of a Split or a Concat): blockIdx.y names the part.
constexpr int MAXPARTS = 8;
struct CopyParts {
    CopyGeom g[MAXPARTS];
    const void* x[MAXPARTS];
    void* y[MAXPARTS];
    uint64_t total[MAXPARTS];
};

template <typename E>
__global__ void __launch_bounds__(256) strided_copy_parts_kernel(const __grid_constant__ CopyParts parts) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    const int part = blockIdx.y;
    const CopyGeom& g = parts.g[part];
    const E* __restrict__ x = static_cast<const E*>(parts.x[part]);
    E* __restrict__ y = static_cast<E*>(parts.y[part]);
    const uint64_t total = parts.total[part];
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += 2 * stride) {
        int64_t xo[2], yo[2];
        const bool second = i + stride < total;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            uint64_t rem = i + u * stride;
            xo[u] = 0, yo[u] = 0;
#pragma unroll
            for (int d = MAXR - 1; d >= 0; --d) {
                if (d < g.rank) {
                    uint64_t c;
                    if (rem < (1ull << 32)) {
                        const uint32_t r32 = static_cast<uint32_t>(rem);
                        c = r32 % g.shape[d];
                        rem = r32 / g.shape[d];
                    } else {
                        c = rem % g.shape[d];
                        rem = rem / g.shape[d];
                    }
                    xo[u] += static_cast<int64_t>(c) * g.xs[d];
                    yo[u] += static_cast<int64_t>(c) * g.ys[d];
                }
            }
        }
        const E v0 = x[xo[0]];
        E v1 = E();
        if (second) v1 = x[xo[1]];
        y[yo[0]] = v0;
        if (second) y[yo[1]] = v1;
    }
}

// y[o][j][k] = data[o][wrap(idx[j])][k]; k runs over `inner` units of E.  An index outside [-dim, dim) writes zeros and
// records DEV_BAD_INDEX in the context's status word.
template <typename E>
__global__ void __launch_bounds__(256) gather_kernel(const E* __restrict__ data, const int64_t* __restrict__ idx,
                                                     E* __restrict__ y, uint64_t total, uint32_t n_idx, uint32_t inner,
                                                     int64_t dim, int32_t* status) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const uint64_t row = i / inner;
        const uint32_t k = static_cast<uint32_t>(i - row * inner);
        const uint64_t o = row / n_idx;
        const uint32_t j = static_cast<uint32_t>(row - o * n_idx);
        int64_t src = __ldg(idx + j);
        if (src < 0) src += dim;
        E v = E();
        if (src >= 0 && src < dim) {
            v = data[(o * static_cast<uint64_t>(dim) + static_cast<uint64_t>(src)) * inner + k];
        } else if (status) {
            atomicCAS(status, DEV_OK, DEV_BAD_INDEX);
        }
        y[i] = v;
    }
}

struct WhereGeom {
    int32_t rank;
    uint32_t shape[MAXR];
    int64_t cs[MAXR], xs[MAXR], ys[MAXR];
};

template <typename E>
__global__ void __launch_bounds__(256) where_kernel(const uint8_t* __restrict__ c, const E* __restrict__ x,
                                                    const E* __restrict__ y, E* __restrict__ out, uint64_t total,
                                                    const WhereGeom g) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        uint64_t rem = i;
        int64_t co = 0, xo = 0, yo = 0;
#pragma unroll
        for (int d = MAXR - 1; d >= 0; --d) {
            if (d < g.rank) {
                const uint64_t q = rem / g.shape[d];
                const uint64_t r = rem - q * g.shape[d];
                rem = q;
                co += static_cast<int64_t>(r) * g.cs[d];
                xo += static_cast<int64_t>(r) * g.xs[d];
                yo += static_cast<int64_t>(r) * g.ys[d];
            }
        }
        out[i] = c[co] ? x[xo] : y[yo];
    }
}

// Same-shape contiguous condition and x, y either the same or one scalar: 16 bytes of x per thread per step.
template <typename E>
__global__ void __launch_bounds__(256) where_fast_kernel(const uint8_t* __restrict__ c, const E* __restrict__ x,
                                                         const E* __restrict__ y, E* __restrict__ out, uint64_t n,
                                                         int y_scalar) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    constexpr int V = 16 / sizeof(E);
    struct alignas(16) Vec { E v[V]; };
    struct alignas(V) Flags { uint8_t f[V]; };
    const uint64_t nvec = n / V;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    const E ys = y_scalar ? y[0] : E();
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        const Flags f = reinterpret_cast<const Flags*>(c)[i];
        const Vec xv = reinterpret_cast<const Vec*>(x)[i];
        Vec yv;
        if (!y_scalar) yv = reinterpret_cast<const Vec*>(y)[i];
        Vec o;
#pragma unroll
        for (int j = 0; j < V; ++j) o.v[j] = f.f[j] ? xv.v[j] : (y_scalar ? ys : yv.v[j]);
        reinterpret_cast<Vec*>(out)[i] = o;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0)
        for (uint64_t i = nvec * V; i < n; ++i) out[i] = c[i] ? x[i] : (y_scalar ? ys : y[i]);
}

template <typename T> struct CmpVec;
template <> struct CmpVec<__half> { static constexpr int V = 8; };
template <> struct CmpVec<float> { static constexpr int V = 4; };
template <> struct CmpVec<long long> { static constexpr int V = 2; };

struct CmpGeom {
    int32_t rank;
    uint32_t shape[MAXR];
    int64_t as[MAXR], bs[MAXR];
};

__device__ __forceinline__ float cmp_ld(const float* p) { return __ldg(p); }
__device__ __forceinline__ float cmp_ld(const __half* p) { return __half2float(__ldg(p)); }
__device__ __forceinline__ long long cmp_ld(const long long* p) { return __ldg(p); }
__device__ __forceinline__ float cmp_val(float v) { return v; }
__device__ __forceinline__ float cmp_val(__half v) { return __half2float(v); }
__device__ __forceinline__ long long cmp_val(long long v) { return v; }

// out[i] = a <op> b as one byte (0 / 1), numpy broadcasting by strides; NaN compares false except for "not equal"
template <typename T>
__global__ void __launch_bounds__(256) compare_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                      uint8_t* __restrict__ out, uint64_t total, int op, const CmpGeom g) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        uint64_t rem = i;
        int64_t ao = 0, bo = 0;
#pragma unroll
        for (int d = MAXR - 1; d >= 0; --d) {
            if (d < g.rank) {
                const uint64_t q = rem / g.shape[d];
                const uint64_t r = rem - q * g.shape[d];
                rem = q;
                ao += static_cast<int64_t>(r) * g.as[d];
                bo += static_cast<int64_t>(r) * g.bs[d];
            }
        }
        const auto x = cmp_ld(a + ao);
        const auto y = cmp_ld(b + bo);
        bool r;
        switch (op) {
            case B200ML_CMP_GT: r = x > y; break;
            case B200ML_CMP_LT: r = x < y; break;
            case B200ML_CMP_GE: r = x >= y; break;
            case B200ML_CMP_LE: r = x <= y; break;
            default: r = x == y; break;
        }
        out[i] = r ? 1 : 0;
    }
}

template <typename A, typename B>
__device__ __forceinline__ bool cmp_apply(int op, A x, B y) {
    switch (op) {
        case B200ML_CMP_GT: return x > y;
        case B200ML_CMP_LT: return x < y;
        case B200ML_CMP_GE: return x >= y;
        case B200ML_CMP_LE: return x <= y;
        default: return x == y;
    }
}

// a contiguous in the output's shape, b the same or one scalar: 16 bytes of a per thread per step
template <typename T>
__global__ void __launch_bounds__(256) compare_fast_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                           uint8_t* __restrict__ out, uint64_t n, int op, int b_scalar) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    constexpr int V = CmpVec<T>::V;
    struct alignas(16) Vec { T v[V]; };
    struct alignas(V) Flags { uint8_t f[V]; };
    const uint64_t nvec = n / V;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    const auto bs = cmp_ld(b);
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        const Vec av = reinterpret_cast<const Vec*>(a)[i];
        Vec bv;
        if (!b_scalar) bv = reinterpret_cast<const Vec*>(b)[i];
        Flags f;
#pragma unroll
        for (int j = 0; j < V; ++j) f.f[j] = cmp_apply(op, cmp_val(av.v[j]), b_scalar ? bs : cmp_val(bv.v[j])) ? 1 : 0;
        reinterpret_cast<Flags*>(out)[i] = f;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0)
        for (uint64_t i = nvec * V; i < n; ++i) out[i] = cmp_apply(op, cmp_ld(a + i), b_scalar ? bs : cmp_ld(b + i)) ? 1 : 0;
}

struct PoolGeom {
    int32_t h, w, oh, ow, kh, kw, sh, sw, pt, pl;
};

__device__ __forceinline__ float pool_ld(const float* p) { return __ldg(p); }
__device__ __forceinline__ float pool_ld(const __half* p) { return __half2float(__ldg(p)); }
__device__ __forceinline__ void pool_st(float* p, float v) { *p = v; }
__device__ __forceinline__ void pool_st(__half* p, float v) { *p = __float2half_rn(v); }

// One thread per output pixel; planes = N * C.  Padding never wins the maximum (it reads as -inf).
template <typename T>
__global__ void __launch_bounds__(256) maxpool2d_kernel(const T* __restrict__ x, T* __restrict__ y, uint64_t total,
                                                        const PoolGeom g) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    const uint32_t opix = static_cast<uint32_t>(g.oh) * g.ow;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const uint64_t plane = i / opix;
        const uint32_t p = static_cast<uint32_t>(i - plane * opix);
        const int oy = p / g.ow, ox = p - oy * g.ow;
        const T* xp = x + plane * static_cast<uint64_t>(g.h) * g.w;
        float m = -CUDART_INF_F;
        for (int ky = 0; ky < g.kh; ++ky) {
            const int iy = oy * g.sh - g.pt + ky;
            if (iy < 0 || iy >= g.h) continue;
            for (int kx = 0; kx < g.kw; ++kx) {
                const int ix = ox * g.sw - g.pl + kx;
                if (ix < 0 || ix >= g.w) continue;
                m = fmaxf(m, pool_ld(xp + iy * g.w + ix));
            }
        }
        pool_st(y + i, m);
    }
}

unsigned grid_for(const b200ml_ctx* ctx, uint64_t total) {
    const uint64_t want = (total + 255) / 256;
    const uint64_t cap = static_cast<uint64_t>(ctx->sm_count) * 32;  // grid-stride beyond 32 blocks of 256 per SM
    return static_cast<unsigned>(want < cap ? (want ? want : 1) : cap);
}

template <typename E>
int launch_copy(const b200ml_ctx* ctx, const void* x, void* y, uint64_t total, const CopyGeom& g, cudaStream_t s) {
    launch_pdl(strided_copy_kernel<E>, dim3(grid_for(ctx, (total + 1) / 2)), dim3(256), 0, s, static_cast<const E*>(x), static_cast<E*>(y), total, g);
    return check_launch("strided_copy");
}

}  // namespace

// 1: the strides are those of a contiguous array of this shape; 0: all zero (one element broadcast); -1: neither
static int stride_kind(int rank, const int64_t* shape, const int64_t* st) {
    bool contiguous = true, scalar = true;
    int64_t acc = 1;
    for (int d = rank - 1; d >= 0; --d) {
        if (shape[d] != 1) {
            contiguous = contiguous && st[d] == acc;
            scalar = scalar && st[d] == 0;
        }
        acc *= shape[d];
    }
    return contiguous ? 1 : (scalar ? 0 : -1);
}

// Coalesces the index space of one copy and picks the unit that moves (1 .. 16 bytes).  *total == 0: nothing to copy.
static int normalize_copy(int elem_bytes, const void* x, const void* y, int rank, const int64_t* shape, const int64_t* xs,
                          const int64_t* ys, CopyGeom* out, uint64_t* total_out, int* unit_out) {
    // drop unit axes, merge neighbours that are contiguous with respect to each other on both sides
    CopyGeom g = {};
    int64_t shp[MAXR];
    int r = 0;
    uint64_t total = 1;
    for (int d = 0; d < rank; ++d) {
        total *= static_cast<uint64_t>(shape[d]);
        if (shape[d] == 1) continue;
        if (r > 0 && g.xs[r - 1] == xs[d] * shape[d] && g.ys[r - 1] == ys[d] * shape[d]) {
            shp[r - 1] *= shape[d];
            g.xs[r - 1] = xs[d];
            g.ys[r - 1] = ys[d];
        } else {
            shp[r] = shape[d];
            g.xs[r] = xs[d];
            g.ys[r] = ys[d];
            ++r;
        }
    }
    *total_out = total;
    if (total == 0) return B200ML_OK;
    if (r == 0) {
        shp[0] = 1, g.xs[0] = 1, g.ys[0] = 1, r = 1;
    }
    for (int d = 0; d < r; ++d) B200ML_REQUIRE(shp[d] < (1ll << 32), "strided_copy: a merged extent exceeds 2^32");
    // widen the unit to 16 bytes when the innermost axis is contiguous on both sides and everything stays aligned
    int unit = elem_bytes;
    const int per16 = 16 / elem_bytes;
    if (g.xs[r - 1] == 1 && g.ys[r - 1] == 1 && shp[r - 1] % per16 == 0 && aligned16(x) && aligned16(y)) {
        bool ok = true;
        for (int d = 0; d < r - 1; ++d) ok = ok && g.xs[d] % per16 == 0 && g.ys[d] % per16 == 0;
        if (ok) {
            unit = 16;
            shp[r - 1] /= per16;
            total /= per16;
            for (int d = 0; d < r - 1; ++d) g.xs[d] /= per16, g.ys[d] /= per16;
        }
    }
    g.rank = r;
    for (int d = 0; d < r; ++d) g.shape[d] = static_cast<uint32_t>(shp[d]);
    *out = g;
    *total_out = total;
    *unit_out = unit;
    return B200ML_OK;
}

static int strided_copy(const b200ml_ctx* ctx, int elem_bytes, const void* x, void* y, int rank, const int64_t* shape,
                 const int64_t* xs, const int64_t* ys, cudaStream_t s) {
    CopyGeom g = {};
    uint64_t total = 0;
    int unit = elem_bytes;
    const int rc = normalize_copy(elem_bytes, x, y, rank, shape, xs, ys, &g, &total, &unit);
    if (rc || total == 0) return rc;
    switch (unit) {
        case 1: return launch_copy<uint8_t>(ctx, x, y, total, g, s);
        case 2: return launch_copy<uint16_t>(ctx, x, y, total, g, s);
        case 4: return launch_copy<uint32_t>(ctx, x, y, total, g, s);
        case 8: return launch_copy<uint64_t>(ctx, x, y, total, g, s);
        default: return launch_copy<uint4>(ctx, x, y, total, g, s);
    }
}

static int gather(const b200ml_ctx* ctx, int elem_bytes, const void* data, const int64_t* indices, void* y, int64_t outer,
           int64_t dim, int64_t inner, int64_t n_idx, cudaStream_t s) {
    uint64_t total = static_cast<uint64_t>(outer) * n_idx * inner;
    if (total == 0) return B200ML_OK;
    const int per16 = 16 / elem_bytes;
    int unit = elem_bytes;
    if (inner % per16 == 0 && aligned16(data) && aligned16(y)) {
        unit = 16;
        inner /= per16;
        total /= per16;
    }
    B200ML_REQUIRE(inner < (1ll << 32) && n_idx < (1ll << 32), "gather: extent exceeds 2^32");
    const unsigned grid = grid_for(ctx, total);
    const uint32_t ni = static_cast<uint32_t>(n_idx), in = static_cast<uint32_t>(inner);
#define B200ML_GATHER(E) \
    launch_pdl(gather_kernel<E>, dim3(grid), dim3(256), 0, s, static_cast<const E*>(data), indices, static_cast<E*>(y), total, ni, in, dim, ctx->status_dev)
    switch (unit) {
        case 1: B200ML_GATHER(uint8_t); break;
        case 2: B200ML_GATHER(uint16_t); break;
        case 4: B200ML_GATHER(uint32_t); break;
        case 8: B200ML_GATHER(uint64_t); break;
        default: B200ML_GATHER(uint4); break;
    }
#undef B200ML_GATHER
    return check_launch("gather");
}

static int where(const b200ml_ctx* ctx, int elem_bytes, const void* cond, const void* x, const void* y, void* out, int rank,
          const int64_t* shape, const int64_t* cs, const int64_t* xs, const int64_t* ys, cudaStream_t s) {
    WhereGeom g = {};
    g.rank = rank;
    uint64_t total = 1;
    for (int d = 0; d < rank; ++d) {
        B200ML_REQUIRE(shape[d] < (1ll << 32), "where: extent exceeds 2^32");
        g.shape[d] = static_cast<uint32_t>(shape[d]);
        g.cs[d] = cs[d], g.xs[d] = xs[d], g.ys[d] = ys[d];
        total *= static_cast<uint64_t>(shape[d]);
    }
    if (total == 0) return B200ML_OK;
    const uint8_t* c = static_cast<const uint8_t*>(cond);
    const int yk = stride_kind(rank, shape, ys);
    if (stride_kind(rank, shape, cs) == 1 && stride_kind(rank, shape, xs) == 1 && yk >= 0 && aligned16(x) && aligned16(out) &&
        (yk == 0 || aligned16(y)) && (reinterpret_cast<uintptr_t>(cond) & 7u) == 0) {
        const unsigned fgrid = grid_for(ctx, total / (16 / elem_bytes) + 1);
        switch (elem_bytes) {
            case 2: launch_pdl(where_fast_kernel<uint16_t>, dim3(fgrid), dim3(256), 0, s, c, (const uint16_t*)x, (const uint16_t*)y, (uint16_t*)out, total, yk == 0); break;
            case 4: launch_pdl(where_fast_kernel<uint32_t>, dim3(fgrid), dim3(256), 0, s, c, (const uint32_t*)x, (const uint32_t*)y, (uint32_t*)out, total, yk == 0); break;
            default: launch_pdl(where_fast_kernel<uint64_t>, dim3(fgrid), dim3(256), 0, s, c, (const uint64_t*)x, (const uint64_t*)y, (uint64_t*)out, total, yk == 0); break;
        }
        return check_launch("where");
    }
    const unsigned grid = grid_for(ctx, total);
    switch (elem_bytes) {
        case 2: launch_pdl(where_kernel<uint16_t>, dim3(grid), dim3(256), 0, s, c, (const uint16_t*)x, (const uint16_t*)y, (uint16_t*)out, total, g); break;
        case 4: launch_pdl(where_kernel<uint32_t>, dim3(grid), dim3(256), 0, s, c, (const uint32_t*)x, (const uint32_t*)y, (uint32_t*)out, total, g); break;
        default: launch_pdl(where_kernel<uint64_t>, dim3(grid), dim3(256), 0, s, c, (const uint64_t*)x, (const uint64_t*)y, (uint64_t*)out, total, g); break;
    }
    return check_launch("where");
}

// ---- Cast between any two of f16, f32, f64, i32, i64, u8 and bool (pure_implementations.py:329-377) -------------
template <typename T> __device__ __forceinline__ double cast_in(T v) { return static_cast<double>(v); }
template <> __device__ __forceinline__ double cast_in<__half>(__half v) { return static_cast<double>(__half2float(v)); }
template <typename T> __device__ __forceinline__ long long cast_in_int(T v) { return static_cast<long long>(v); }
template <> __device__ __forceinline__ long long cast_in_int<__half>(__half v) { return static_cast<long long>(__half2float(v)); }

template <typename S> struct IsFloat { static constexpr bool value = false; };
template <> struct IsFloat<__half> { static constexpr bool value = true; };
template <> struct IsFloat<float> { static constexpr bool value = true; };
template <> struct IsFloat<double> { static constexpr bool value = true; };

struct BoolTag {};  // destination "bool": x != 0 as one byte

template <typename D, typename S>
__device__ __forceinline__ D cast_one(S v) {
    if constexpr (IsFloat<D>::value) {
        // integers go through long long so that int64 keeps every bit a double can hold; floats through double
        if constexpr (IsFloat<S>::value) {
            const double d = cast_in(v);
            if constexpr (sizeof(D) == 2) return __float2half_rn(static_cast<float>(d));
            else return static_cast<D>(d);
        } else {
            const long long q = static_cast<long long>(v);
            if constexpr (sizeof(D) == 2) return __float2half_rn(static_cast<float>(q));
            else return static_cast<D>(q);
        }
    } else {
        if constexpr (IsFloat<S>::value) return static_cast<D>(cast_in_int(v));  // truncation toward zero
        else return static_cast<D>(v);
    }
}

template <typename S, typename D, bool TO_BOOL>
__global__ void __launch_bounds__(256) cast_any_kernel(const S* __restrict__ x, D* __restrict__ y, uint64_t n) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const S v = x[i];
        if constexpr (TO_BOOL) {
            bool nz;
            if constexpr (IsFloat<S>::value) nz = cast_in(v) != 0.0;
            else nz = v != 0;
            y[i] = nz ? 1 : 0;
        } else {
            y[i] = cast_one<D, S>(v);
        }
    }
}

template <typename S>
static int cast_from(const b200ml_ctx* ctx, int dst, const S* x, void* y, uint64_t n, cudaStream_t s) {
    const unsigned grid = grid_for(ctx, n);
    switch (dst) {
        case B200ML_F16: launch_pdl(cast_any_kernel<S, __half, false>, dim3(grid), dim3(256), 0, s, x, static_cast<__half*>(y), n); break;
        case B200ML_F32: launch_pdl(cast_any_kernel<S, float, false>, dim3(grid), dim3(256), 0, s, x, static_cast<float*>(y), n); break;
        case B200ML_F64: launch_pdl(cast_any_kernel<S, double, false>, dim3(grid), dim3(256), 0, s, x, static_cast<double*>(y), n); break;
        case B200ML_I32: launch_pdl(cast_any_kernel<S, int32_t, false>, dim3(grid), dim3(256), 0, s, x, static_cast<int32_t*>(y), n); break;
        case B200ML_I64: launch_pdl(cast_any_kernel<S, long long, false>, dim3(grid), dim3(256), 0, s, x, static_cast<long long*>(y), n); break;
        case B200ML_U8: launch_pdl(cast_any_kernel<S, uint8_t, false>, dim3(grid), dim3(256), 0, s, x, static_cast<uint8_t*>(y), n); break;
        default: launch_pdl(cast_any_kernel<S, uint8_t, true>, dim3(grid), dim3(256), 0, s, x, static_cast<uint8_t*>(y), n); break;
    }
    return check_launch("cast");
}

int cast_any(const b200ml_ctx* ctx, int src, int dst, const void* x, void* y, int64_t n, cudaStream_t s) {
    const uint64_t un = static_cast<uint64_t>(n);
    switch (src) {
        case B200ML_F16: return cast_from(ctx, dst, static_cast<const __half*>(x), y, un, s);
        case B200ML_F32: return cast_from(ctx, dst, static_cast<const float*>(x), y, un, s);
        case B200ML_F64: return cast_from(ctx, dst, static_cast<const double*>(x), y, un, s);
        case B200ML_I32: return cast_from(ctx, dst, static_cast<const int32_t*>(x), y, un, s);
        case B200ML_I64: return cast_from(ctx, dst, static_cast<const long long*>(x), y, un, s);
        default: return cast_from(ctx, dst, static_cast<const uint8_t*>(x), y, un, s);  // u8 and bool read alike
    }
}

static int compare(const b200ml_ctx* ctx, int kind, int op, const void* a, const void* b, void* out, int rank,
                   const int64_t* shape, const int64_t* as, const int64_t* bs, cudaStream_t s) {
    CmpGeom g = {};
    g.rank = rank;
    uint64_t total = 1;
    for (int d = 0; d < rank; ++d) {
        B200ML_REQUIRE(shape[d] < (1ll << 32), "compare: extent exceeds 2^32");
        g.shape[d] = static_cast<uint32_t>(shape[d]);
        g.as[d] = as[d], g.bs[d] = bs[d];
        total *= static_cast<uint64_t>(shape[d]);
    }
    if (total == 0) return B200ML_OK;
    uint8_t* o = static_cast<uint8_t*>(out);
    const int bk = stride_kind(rank, shape, bs);
    if (stride_kind(rank, shape, as) == 1 && bk >= 0 && aligned16(a) && (bk == 0 || aligned16(b)) &&
        (reinterpret_cast<uintptr_t>(out) & 7u) == 0) {
        const int v = kind == B200ML_F16 ? 8 : (kind == B200ML_F32 ? 4 : 2);
        const unsigned fgrid = grid_for(ctx, total / v + 1);
        if (kind == B200ML_F16)
            launch_pdl(compare_fast_kernel<__half>, dim3(fgrid), dim3(256), 0, s, (const __half*)a, (const __half*)b, o, total, op, bk == 0);
        else if (kind == B200ML_F32)
            launch_pdl(compare_fast_kernel<float>, dim3(fgrid), dim3(256), 0, s, (const float*)a, (const float*)b, o, total, op, bk == 0);
        else
            launch_pdl(compare_fast_kernel<long long>, dim3(fgrid), dim3(256), 0, s, (const long long*)a, (const long long*)b, o, total, op, bk == 0);
        return check_launch("compare");
    }
    const unsigned grid = grid_for(ctx, total);
    if (kind == B200ML_F16)
        launch_pdl(compare_kernel<__half>, dim3(grid), dim3(256), 0, s, (const __half*)a, (const __half*)b, o, total, op, g);
    else if (kind == B200ML_F32)
        launch_pdl(compare_kernel<float>, dim3(grid), dim3(256), 0, s, (const float*)a, (const float*)b, o, total, op, g);
    else
        launch_pdl(compare_kernel<long long>, dim3(grid), dim3(256), 0, s, (const long long*)a, (const long long*)b, o, total, op, g);
    return check_launch("compare");
}

static int maxpool2d(const b200ml_ctx* ctx, int dtype, const void* x, void* y, int64_t planes, const PoolGeom& g, cudaStream_t s) {
    const uint64_t total = static_cast<uint64_t>(planes) * g.oh * g.ow;
    if (total == 0) return B200ML_OK;
    const unsigned grid = grid_for(ctx, total);
    if (dtype == B200ML_F16)
        launch_pdl(maxpool2d_kernel<__half>, dim3(grid), dim3(256), 0, s, static_cast<const __half*>(x), static_cast<__half*>(y), total, g);
    else
        launch_pdl(maxpool2d_kernel<float>, dim3(grid), dim3(256), 0, s, static_cast<const float*>(x), static_cast<float*>(y), total, g);
    return check_launch("maxpool2d");
}

namespace {
template <typename E>
int launch_parts(const b200ml_ctx* ctx, const CopyParts& parts, int nparts, uint64_t largest, cudaStream_t s) {
    const dim3 grid(grid_for(ctx, (largest + 1) / 2), (unsigned)nparts);
    launch_pdl(strided_copy_parts_kernel<E>, grid, dim3(256), 0, s, parts);
    return check_launch("strided_copy_parts");
}
}  // namespace

// Several copies of the same element size at once.  One launch when every part moves the same unit, else one per part.
static int strided_copy_parts(const b200ml_ctx* ctx, int elem_bytes, int nparts, const void* const* xs_, void* const* ys_,
                              int rank, const int64_t* shapes, const int64_t* x_strides, const int64_t* y_strides,
                              cudaStream_t s) {
    CopyParts parts = {};
    int units[MAXPARTS];
    uint64_t largest = 0;
    int live = 0;
    bool same = true;
    for (int p = 0; p < nparts; ++p) {
        CopyGeom g = {};
        uint64_t total = 0;
        int unit = elem_bytes;
        const int rc = normalize_copy(elem_bytes, xs_[p], ys_[p], rank, shapes + p * rank, x_strides + p * rank,
                                      y_strides + p * rank, &g, &total, &unit);
        if (rc) return rc;
        if (total == 0) continue;
        parts.g[live] = g, parts.x[live] = xs_[p], parts.y[live] = ys_[p], parts.total[live] = total, units[live] = unit;
        same = same && unit == units[0];
        largest = total > largest ? total : largest;
        ++live;
    }
    if (live == 0) return B200ML_OK;
    if (!same || live == 1) {
        for (int p = 0; p < nparts; ++p) {
            const int rc = strided_copy(ctx, elem_bytes, xs_[p], ys_[p], rank, shapes + p * rank, x_strides + p * rank,
                                        y_strides + p * rank, s);
            if (rc) return rc;
        }
        return B200ML_OK;
    }
    switch (units[0]) {
        case 1: return launch_parts<uint8_t>(ctx, parts, live, largest, s);
        case 2: return launch_parts<uint16_t>(ctx, parts, live, largest, s);
        case 4: return launch_parts<uint32_t>(ctx, parts, live, largest, s);
        case 8: return launch_parts<uint64_t>(ctx, parts, live, largest, s);
        default: return launch_parts<uint4>(ctx, parts, live, largest, s);
    }
}
}  // namespace b200ml

using namespace b200ml;

extern "C" {

int b200ml_strided_copy(b200ml_ctx* ctx, int32_t elem_bytes, const void* x, void* y, int32_t rank, const int64_t* shape,
                        const int64_t* x_strides, const int64_t* y_strides, b200ml_stream stream) {
    B200ML_REQUIRE(ctx, "strided_copy: null context");
    B200ML_REQUIRE(elem_bytes == 1 || elem_bytes == 2 || elem_bytes == 4 || elem_bytes == 8,
                   "strided_copy: element size %d not supported", elem_bytes);
    B200ML_REQUIRE(rank >= 0 && rank <= MAXR, "strided_copy: rank %d not in [0, 6]", rank);
    B200ML_REQUIRE(rank == 0 || (shape && x_strides && y_strides), "strided_copy: null shape or strides");
    for (int d = 0; d < rank; ++d) {
        B200ML_REQUIRE(shape[d] >= 0, "strided_copy: negative extent");
        B200ML_REQUIRE(x_strides[d] >= 0 && y_strides[d] >= 0, "strided_copy: negative stride");
        B200ML_REQUIRE(y_strides[d] > 0 || shape[d] <= 1, "strided_copy: destination stride 0 on an axis of extent %lld",
                       (long long)shape[d]);
    }
    B200ML_REQUIRE(x && y, "strided_copy: null tensor");
    DeviceGuard guard(ctx->device);
    return strided_copy(ctx, elem_bytes, x, y, rank, shape, x_strides, y_strides, static_cast<cudaStream_t>(stream));
}

int b200ml_strided_copy_parts(b200ml_ctx* ctx, int32_t elem_bytes, int32_t nparts, const void* const* xs, void* const* ys,
                              int32_t rank, const int64_t* shapes, const int64_t* x_strides, const int64_t* y_strides,
                              b200ml_stream stream) {
    B200ML_REQUIRE(ctx, "strided_copy_parts: null context");
    B200ML_REQUIRE(elem_bytes == 1 || elem_bytes == 2 || elem_bytes == 4 || elem_bytes == 8,
                   "strided_copy_parts: element size %d not supported", elem_bytes);
    B200ML_REQUIRE(nparts >= 1 && nparts <= MAXPARTS, "strided_copy_parts: %d parts, 1 to 8 are taken", nparts);
    B200ML_REQUIRE(rank >= 1 && rank <= MAXR, "strided_copy_parts: rank %d not in [1, 6]", rank);
    B200ML_REQUIRE(xs && ys && shapes && x_strides && y_strides, "strided_copy_parts: null argument");
    for (int p = 0; p < nparts; ++p) {
        B200ML_REQUIRE(xs[p] && ys[p], "strided_copy_parts: null tensor in part %d", p);
        for (int d = 0; d < rank; ++d) {
            const int64_t ext = shapes[p * rank + d], xst = x_strides[p * rank + d], yst = y_strides[p * rank + d];
            B200ML_REQUIRE(ext >= 0 && xst >= 0 && yst >= 0, "strided_copy_parts: negative extent or stride");
            B200ML_REQUIRE(yst > 0 || ext <= 1, "strided_copy_parts: destination stride 0 on an axis of extent %lld", (long long)ext);
        }
    }
    DeviceGuard guard(ctx->device);
    return strided_copy_parts(ctx, elem_bytes, nparts, xs, ys, rank, shapes, x_strides, y_strides, static_cast<cudaStream_t>(stream));
}

int b200ml_gather(b200ml_ctx* ctx, int32_t elem_bytes, const void* data, const int64_t* indices, void* y, int64_t outer,
                  int64_t axis_dim, int64_t inner, int64_t n_indices, b200ml_stream stream) {
    B200ML_REQUIRE(ctx, "gather: null context");
    B200ML_REQUIRE(elem_bytes == 1 || elem_bytes == 2 || elem_bytes == 4 || elem_bytes == 8,
                   "gather: element size %d not supported", elem_bytes);
    B200ML_REQUIRE(outer >= 0 && axis_dim >= 0 && inner >= 0 && n_indices >= 0, "gather: negative extent");
    if (outer == 0 || inner == 0 || n_indices == 0) return B200ML_OK;
    B200ML_REQUIRE(axis_dim > 0, "gather: indices into an empty axis");
    B200ML_REQUIRE(data && indices && y, "gather: null tensor");
    DeviceGuard guard(ctx->device);
    return gather(ctx, elem_bytes, data, indices, y, outer, axis_dim, inner, n_indices, static_cast<cudaStream_t>(stream));
}

int b200ml_where(b200ml_ctx* ctx, int32_t elem_bytes, const void* condition, const void* x, const void* y, void* out,
                 int32_t rank, const int64_t* shape, const int64_t* c_strides, const int64_t* x_strides,
                 const int64_t* y_strides, b200ml_stream stream) {
    B200ML_REQUIRE(ctx, "where: null context");
    B200ML_REQUIRE(elem_bytes == 2 || elem_bytes == 4 || elem_bytes == 8, "where: element size %d not supported", elem_bytes);
    B200ML_REQUIRE(rank >= 0 && rank <= MAXR, "where: rank %d not in [0, 6]", rank);
    B200ML_REQUIRE(rank == 0 || (shape && c_strides && x_strides && y_strides), "where: null shape or strides");
    for (int d = 0; d < rank; ++d) {
        B200ML_REQUIRE(shape[d] >= 0, "where: negative extent");
        B200ML_REQUIRE(c_strides[d] >= 0 && x_strides[d] >= 0 && y_strides[d] >= 0, "where: negative stride");
    }
    B200ML_REQUIRE(condition && x && y && out, "where: null tensor");
    DeviceGuard guard(ctx->device);
    return where(ctx, elem_bytes, condition, x, y, out, rank, shape, c_strides, x_strides, y_strides,
                 static_cast<cudaStream_t>(stream));
}

int b200ml_compare(b200ml_ctx* ctx, int32_t dtype, int32_t op, const void* a, const void* b, void* out, int32_t rank,
                   const int64_t* shape, const int64_t* a_strides, const int64_t* b_strides, b200ml_stream stream) {
    B200ML_REQUIRE(ctx, "compare: null context");
    B200ML_REQUIRE(dtype == B200ML_F16 || dtype == B200ML_F32 || dtype == B200ML_I64, "compare: unknown dtype");
    B200ML_REQUIRE(op >= B200ML_CMP_EQ && op <= B200ML_CMP_LE, "compare: unknown operator %d", op);
    B200ML_REQUIRE(rank >= 0 && rank <= MAXR, "compare: rank %d not in [0, 6]", rank);
    B200ML_REQUIRE(rank == 0 || (shape && a_strides && b_strides), "compare: null shape or strides");
    for (int d = 0; d < rank; ++d) {
        B200ML_REQUIRE(shape[d] >= 0, "compare: negative extent");
        B200ML_REQUIRE(a_strides[d] >= 0 && b_strides[d] >= 0, "compare: negative stride");
    }
    B200ML_REQUIRE(a && b && out, "compare: null tensor");
    DeviceGuard guard(ctx->device);
    return compare(ctx, dtype, op, a, b, out, rank, shape, a_strides, b_strides, static_cast<cudaStream_t>(stream));
}

int b200ml_maxpool2d(b200ml_ctx* ctx, int32_t dtype, const void* x, void* y, int64_t planes, int64_t h, int64_t w,
                     int32_t kh, int32_t kw, int32_t stride_h, int32_t stride_w, int32_t pad_top, int32_t pad_left,
                     int32_t pad_bottom, int32_t pad_right, b200ml_stream stream) {
    B200ML_REQUIRE(ctx, "maxpool2d: null context");
    B200ML_REQUIRE(dtype == B200ML_F16 || dtype == B200ML_F32, "maxpool2d: unknown dtype");
    B200ML_REQUIRE(planes >= 0 && h > 0 && w > 0 && h < (1 << 30) && w < (1 << 30), "maxpool2d: bad extent");
    B200ML_REQUIRE(kh > 0 && kw > 0 && stride_h > 0 && stride_w > 0, "maxpool2d: kernel and strides must be positive");
    B200ML_REQUIRE(pad_top >= 0 && pad_left >= 0 && pad_bottom >= 0 && pad_right >= 0, "maxpool2d: negative padding");
    B200ML_REQUIRE(pad_top < kh && pad_bottom < kh && pad_left < kw && pad_right < kw,
                   "maxpool2d: padding must be smaller than the kernel (a window may not lie in the padding alone)");
    const int64_t oh = (h + pad_top + pad_bottom - kh) / stride_h + 1, ow = (w + pad_left + pad_right - kw) / stride_w + 1;
    B200ML_REQUIRE(h + pad_top + pad_bottom >= kh && w + pad_left + pad_right >= kw, "maxpool2d: kernel larger than the padded image");
    if (planes == 0) return B200ML_OK;
    B200ML_REQUIRE(x && y, "maxpool2d: null tensor");
    DeviceGuard guard(ctx->device);
    PoolGeom g = {(int32_t)h, (int32_t)w, (int32_t)oh, (int32_t)ow, kh, kw, stride_h, stride_w, pad_top, pad_left};
    return maxpool2d(ctx, dtype, x, y, planes, g, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
