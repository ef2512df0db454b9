// Tiled kernels for the gather side of QK / AV (head_dim 32, m <= 48):
//
//   tiled_sum   out[i,:] = sum_j W[i,j] * X[idx[i,j],:]     AV forward, d_query
//   tiled_dot   out[i,j] = <X[idx[i,j],:], Y[i,:]>          QK forward, d_attn
//
// Every WARP works on its own: it takes a tile of 8 consecutive rows (one AutoFocusFormer
// cluster) of one batch element, reads the tile's int64 neighbour indices once (cp.async into
// shared memory) and then serves all heads from them.  For a head it stages each distinct
// neighbour row ONCE in shared memory (cp.async, 16-byte chunks XOR-swizzled by row) and
// multiplies the 8 rows of the tile against the staged rows with a register-tiled product on
// the FP32 pipes (two-wide FMAs).  There is no block-level synchronisation; latency is hidden by
// running about twenty such warps per SM (11 KB of shared memory each) and by L2 prefetches of
// the next tile's index and weight lines.
//
// Tiles whose 8 rows are identical (the tokens of a cluster share their neighbourhood) need no
// de-duplication: the slot of a neighbour is its column.  Otherwise the warp de-duplicates the
// 8 x m indices with a bitmap over token ids (slots ascend with the token id, which fixes the
// summation order) and spreads the weights into a dense [8 x U] matrix, 48 distinct neighbours
// at a time.
//
// The reference gives each output element a thread that re-gathers its neighbour rows from L2
// (clusten/src/clustenav_cuda_kernel.cu:18-50, clustenqk_cuda_kernel.cu:18-49).
#include <limits.h>
#include <type_traits>

#include "tiled.cuh"

namespace clusten {

__device__ int g_device_status = 0;   // bits of kErr*, see read_device_status

namespace {

constexpr int kT = 8;              // rows per tile
constexpr int kC = 32;             // channels per head
constexpr int kMmax = 48;          // neighbours per row handled here
constexpr int kE = kT * kMmax;     // edges per tile
constexpr int kUC = 48;            // distinct neighbour rows per stage
constexpr int kWLD = 52;           // row stride (floats) of the score tile
constexpr int kWLD2 = 100;         // row stride (floats) of the weight tile, every weight stored twice
constexpr int kYLD = 36;           // row stride (floats) of the fp32 Y tile
constexpr int kBMW = 256;          // bitmap words: token ids of a tile may span 8192
constexpr int kWarps = 4;          // warps per CTA (independent of each other)
constexpr int kEPL = kE / 32;      // edges per lane
constexpr unsigned kFull = 0xffffffffu;
constexpr unsigned short kSkip = 0xffffu;

// ----------------------------------------------------------------------------- shared memory (per warp)
//   X    neighbour rows [48][32] fp32; its front doubles as landing area of the tile's int64 indices
//   Xraw (16-bit inputs) the rows as loaded, converted to fp32 into X
//   Op   tiled_sum: weight tile [8][kWLD2];  tiled_dot: Y tile [8][kYLD] + score tile [8][kWLD];
//        doubles as bitmap scratch while a tile is de-duplicated
//   lut  edge -> slot,  uniq  slot -> source row
template <typename T, int MODE> struct WarpSmem {
    static constexpr bool kIsFloat = std::is_same<T, float>::value;
    static constexpr int kX = kUC * kC * 4;
    static constexpr int kXraw = kIsFloat ? 0 : kUC * kC * (int)sizeof(T);
    static constexpr int kOp = MODE == 0 ? kT * kWLD2 * 4 : (kT * kYLD + kT * kWLD) * 4;
    static constexpr int kLut = kE * 2;
    static constexpr int kTotal = kX + kXraw + kOp + 2 * kLut;
};
static_assert(kBMW * 4 + kBMW * 2 + (kE / 32) * 4 <= (kT * kYLD + kT * kWLD) * 4, "bitmap scratch must fit in Op");

// ----------------------------------------------------------------------------- PTX helpers
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16_ca(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(dst)), "l"(src));
}
__device__ __forceinline__ void cp_async8_ca(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(smem_u32(dst)), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];\n" ::"l"(p)); }

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const __half* p) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&r.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&r.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xffff0000u),
                       __uint_as_float(r.y << 16), __uint_as_float(r.y & 0xffff0000u));
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__half* p, float4 v) {
    const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
    uint2 r;
    r.x = *reinterpret_cast<const unsigned*>(&a);
    r.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = r;
}
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 r;
    r.x = *reinterpret_cast<const unsigned*>(&a);
    r.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = r;
}

// ----------------------------------------------------------------------------- products
// acc[a] += Wd[2qi+a][u] * Xs[u][4ci..4ci+3] for u < rows8 (multiple of 8).  Wd holds every weight
// twice (row stride kWLD2) so that one two-wide FMA updates a channel pair; Xs chunks are swizzled
// by the row number, swz[k] = ((ci ^ k) << 2).
__device__ __forceinline__ void sum_product(const float* __restrict__ Wd, const float* __restrict__ Xs, int rows8,
                                            int qi, const int (&swz)[8], float2 (&acc)[2][2]) {
    const float* w0p = Wd + (2 * qi) * kWLD2;
    const float* w1p = w0p + kWLD2;
    for (int u = 0; u < rows8; u += 8) {
        const float* xr = Xs + u * kC;
#pragma unroll
        for (int k = 0; k < 8; k += 2) {
            const float4 wa = *reinterpret_cast<const float4*>(w0p + 2 * (u + k));   // {w_k, w_k, w_k+1, w_k+1}
            const float4 wb = *reinterpret_cast<const float4*>(w1p + 2 * (u + k));
            const float4 x0 = *reinterpret_cast<const float4*>(xr + k * kC + swz[k]);
            const float4 x1 = *reinterpret_cast<const float4*>(xr + (k + 1) * kC + swz[k + 1]);
            acc[0][0] = __ffma2_rn(make_float2(wa.x, wa.y), make_float2(x0.x, x0.y), acc[0][0]);
            acc[0][1] = __ffma2_rn(make_float2(wa.x, wa.y), make_float2(x0.z, x0.w), acc[0][1]);
            acc[1][0] = __ffma2_rn(make_float2(wb.x, wb.y), make_float2(x0.x, x0.y), acc[1][0]);
            acc[1][1] = __ffma2_rn(make_float2(wb.x, wb.y), make_float2(x0.z, x0.w), acc[1][1]);
            acc[0][0] = __ffma2_rn(make_float2(wa.z, wa.w), make_float2(x1.x, x1.y), acc[0][0]);
            acc[0][1] = __ffma2_rn(make_float2(wa.z, wa.w), make_float2(x1.z, x1.w), acc[0][1]);
            acc[1][0] = __ffma2_rn(make_float2(wb.z, wb.w), make_float2(x1.x, x1.y), acc[1][0]);
            acc[1][1] = __ffma2_rn(make_float2(wb.z, wb.w), make_float2(x1.z, x1.w), acc[1][1]);
        }
    }
}

// Sb[2qi+a][8k+ui] = <Ys[2qi+a][:], Xs[8k+ui][:]> for k < kmax; two-wide FMAs over channel pairs
__device__ __forceinline__ void dot_product(const float* __restrict__ Ys, const float* __restrict__ Xs,
                                            float* __restrict__ Sb, int kmax, int qi, int ui) {
    constexpr int K = kUC / 8;
    float2 acc[2][K];
#pragma unroll
    for (int k = 0; k < K; ++k) acc[0][k] = acc[1][k] = make_float2(0.f, 0.f);
    const float* y0p = Ys + (2 * qi) * kYLD;
    const float* y1p = y0p + kYLD;
#pragma unroll 2
    for (int c4 = 0; c4 < kC / 4; ++c4) {
        const float4 y0 = *reinterpret_cast<const float4*>(y0p + c4 * 4);
        const float4 y1 = *reinterpret_cast<const float4*>(y1p + c4 * 4);
        const int off = (c4 ^ ui) << 2;
#pragma unroll
        for (int k = 0; k < K; ++k) {
            if (k < kmax) {
                const float4 x = *reinterpret_cast<const float4*>(Xs + (8 * k + ui) * kC + off);
                acc[0][k] = __ffma2_rn(make_float2(y0.x, y0.y), make_float2(x.x, x.y), acc[0][k]);
                acc[0][k] = __ffma2_rn(make_float2(y0.z, y0.w), make_float2(x.z, x.w), acc[0][k]);
                acc[1][k] = __ffma2_rn(make_float2(y1.x, y1.y), make_float2(x.x, x.y), acc[1][k]);
                acc[1][k] = __ffma2_rn(make_float2(y1.z, y1.w), make_float2(x.z, x.w), acc[1][k]);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < K; ++k) {
        if (k < kmax) {
            Sb[(2 * qi) * kWLD + 8 * k + ui] = acc[0][k].x + acc[0][k].y;
            Sb[(2 * qi + 1) * kWLD + 8 * k + ui] = acc[1][k].x + acc[1][k].y;
        }
    }
}

// ----------------------------------------------------------------------------- producer: tile analysis
// Are the 8 rows of the tile identical, in range, and the tile complete?  One warp.
__device__ __forceinline__ bool rows_identical(const long long* ring, int E, int m, int n, bool complete,
                                               int lane) {
    const int4* r = reinterpret_cast<const int4*>(ring);      // {lo, hi, lo, hi} of two entries
    bool same = complete && (m & 7) == 0;
    int col = (2 * lane) % m;
    const int col_step = 64 % m;
    for (int x = lane; 2 * x < E; x += 32) {
        const int4 v = r[x];
        const int4 ref = r[col >> 1];
        if (v.x != ref.x || v.z != ref.z || (v.y | v.w) != 0 || (unsigned)v.x >= (unsigned)n ||
            (unsigned)v.z >= (unsigned)n)
            same = false;
        col += col_step;
        if (col >= m) col -= m;
    }
    return __all_sync(kFull, same);
}

// De-duplicate the tile's indices: tok / uniq in the scratch, edge -> slot in lut.  Returns U; *rowdup
// tells whether some row names a neighbour more than once.  One warp.
struct DedupScratch {
    unsigned short* tok;     // [kE] source row of each edge, kSkip = none
    unsigned short* uniq;    // [kE] slot -> source row
    unsigned* bm;            // [kBMW]
    unsigned short* pre;     // [kBMW]
    unsigned* rowbm;         // [kE / 32]
};
__device__ int dedup_tile(const DedupScratch ps_, const long long* ring, unsigned short* lut, int E, int m, int i0,
                          int n, bool want_rowdup, bool* rowdup, int lane) {
    const DedupScratch* ps = &ps_;
    int lo = INT_MAX, hi = -1;
    for (int x = lane; x < E; x += 32) {
        const long long v = ring[x];
        const int q = x / m;
        unsigned short t = kSkip;
        if (i0 + q < n && v >= 0 && v < n) {
            t = (unsigned short)v;
            lo = min(lo, (int)v);
            hi = max(hi, (int)v);
        }
        ps->tok[x] = t;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        lo = min(lo, __shfl_xor_sync(kFull, lo, o));
        hi = max(hi, __shfl_xor_sync(kFull, hi, o));
    }
    *rowdup = false;
    __syncwarp();
    if (hi < 0) {
        for (int x = lane; x < E; x += 32) lut[x] = kSkip;
        __syncwarp();
        return 0;
    }
    const int w0 = lo >> 5;
    const int words = (hi >> 5) - w0 + 1;
    if (words > kBMW) {                       // ids too spread out: one slot per edge
        for (int x = lane; x < E; x += 32) {
            const unsigned short t = ps->tok[x];
            lut[x] = t != kSkip ? (unsigned short)x : kSkip;
            ps->uniq[x] = t;
        }
        __syncwarp();
        return E;
    }
    for (int w = lane; w < words; w += 32) ps->bm[w] = 0u;
    __syncwarp();
    for (int x = lane; x < E; x += 32) {
        const unsigned short t = ps->tok[x];
        if (t != kSkip) atomicOr(&ps->bm[(t >> 5) - w0], 1u << (t & 31));
    }
    __syncwarp();
    const int per = (words + 31) >> 5;
    const int a = min(lane * per, words), b = min(a + per, words);
    int local = 0;
    for (int w = a; w < b; ++w) local += __popc(ps->bm[w]);
    int incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(kFull, incl, o);
        if (lane >= o) incl += y;
    }
    const int U = __shfl_sync(kFull, incl, 31);
    int run = incl - local;
    for (int w = a; w < b; ++w) {
        ps->pre[w] = (unsigned short)run;
        run += __popc(ps->bm[w]);
    }
    __syncwarp();
    for (int x = lane; x < E; x += 32) {
        const unsigned short t = ps->tok[x];
        if (t != kSkip) {
            const int w = (t >> 5) - w0;
            const int s = ps->pre[w] + __popc(ps->bm[w] & ((1u << (t & 31)) - 1u));
            lut[x] = (unsigned short)s;
            ps->uniq[s] = t;
        } else {
            lut[x] = kSkip;
        }
    }
    __syncwarp();
    if (want_rowdup && U < E) {               // does a row hit one slot twice?
        bool seen = false;
        const int rw = (U + 31) >> 5;
        for (int q = 0; q < kT; ++q) {
            if (lane < rw) ps->rowbm[lane] = 0u;
            __syncwarp();
            for (int jj = lane; jj < m; jj += 32) {
                const unsigned short s = lut[q * m + jj];
                if (s != kSkip) {
                    const unsigned bit = 1u << (s & 31);
                    if (atomicOr(&ps->rowbm[s >> 5], bit) & bit) seen = true;
                }
            }
            __syncwarp();
        }
        *rowdup = __any_sync(kFull, seen);
    }
    return U;
}

// ----------------------------------------------------------------------------- the kernel
// MODE 0: tiled_sum (A = W [bb, n, m]),  MODE 1: tiled_dot (A = Y [bb, n, 32]); X = [bb, n, 32]
template <typename T, int MODE>
__global__ void __launch_bounds__(32 * kWarps, 5)
gather_tiles_kernel(const T* __restrict__ A, const T* __restrict__ X, const int64_t* __restrict__ idx,
                    T* __restrict__ out, int batch, int heads, int n, int m, int tiles) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    using WS = WarpSmem<T, MODE>;
    constexpr bool kIsFloat = WS::kIsFloat;
    constexpr int kPer = 16 / (int)sizeof(T);          // elements per 16-byte piece
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int qi = lane >> 3, ci = lane & 7;
    unsigned char* base = smem_raw + size_t(warp) * WS::kTotal;
    float* Xs = reinterpret_cast<float*>(base);
    T* Xraw = reinterpret_cast<T*>(base + WS::kX);
    float* Op = reinterpret_cast<float*>(base + WS::kX + WS::kXraw);
    unsigned short* lut = reinterpret_cast<unsigned short*>(base + WS::kX + WS::kXraw + WS::kOp);
    unsigned short* uniq = lut + kE;
    float* Wd = Op;                                     // MODE 0
    float* Ys = Op;                                     // MODE 1
    float* Sb = Op + kT * kYLD;                         // MODE 1
    long long* ring = reinterpret_cast<long long*>(Xs);               // first 3 KB of X
    DedupScratch ds;
    ds.tok = reinterpret_cast<unsigned short*>(base + kE * 8);        // behind the landed indices
    ds.uniq = uniq;
    ds.bm = reinterpret_cast<unsigned*>(Op);
    ds.pre = reinterpret_cast<unsigned short*>(ds.bm + kBMW);
    ds.rowbm = reinterpret_cast<unsigned*>(ds.pre + kBMW);

    const int E = kT * m;
    const int m4 = m >> 2;
    int swz[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) swz[k] = (ci ^ k) << 2;
    const int sw_even = (ci ^ qi) << 2, sw_odd = sw_even ^ 16;   // swizzle of row qi + 4k, k even / odd
    // piece z = lane + 32k of a [8][m] tile -> (row, 4-element piece); edge x = lane + 32k -> its row
    int wq[3], wc[3];
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        const int z = lane + 32 * k;
        const int d = m4 > 0 ? m4 : 1;
        wq[k] = z / d;
        wc[k] = z - wq[k] * d;
    }
    unsigned long long qpack = 0ull;                    // 3 bits per edge: its row
#pragma unroll
    for (int k = 0; k < kEPL; ++k) qpack |= (unsigned long long)(((lane + 32 * k) / m) & 7) << (3 * k);

    const long long total = (long long)batch * tiles;
    const long long nwarps = (long long)gridDim.x * kWarps;
    for (long long task = (long long)blockIdx.x * kWarps + warp; task < total; task += nwarps) {
        const int b = (int)(task / tiles);
        const int tile = (int)(task - (long long)b * tiles);
        const int i0 = tile * kT;
        const bool complete = i0 + kT <= n;
        const int64_t* src = idx + ((long long)b * n + i0) * m;
        // ---- warm the L2 for this warp's next tile: its index rows and its weight / Y rows
        {
            const long long nx = task + nwarps;
            if (nx < total) {
                const int nb = (int)(nx / tiles);
                const int ni0 = (int)(nx - (long long)nb * tiles) * kT;
                if (lane * 16 < E) prefetch_l2(idx + ((long long)nb * n + ni0) * m + lane * 16);
                const int arow = MODE == 0 ? m : kC;               // elements per row of A
                const int abytes = kT * arow * (int)sizeof(T);
                for (int g = 0; g < heads; ++g)
                    if (lane * 128 < abytes)
                        prefetch_l2(reinterpret_cast<const char*>(A + (((long long)nb * heads + g) * n + ni0) * arow) +
                                    lane * 128);
            }
        }
        // ---- the tile's indices
        __syncwarp();
        if (complete && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
            for (int x = 2 * lane; x < E; x += 64) cp_async16_ca(ring + x, src + x);
        } else {
            const int valid = min(kT, n - i0) * m;
            for (int x = lane; x < E; x += 32) {
                if (x < valid) cp_async8_ca(ring + x, src + x);
                else ring[x] = -1;
            }
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncwarp();
        const bool identical = rows_identical(ring, E, m, n, complete, lane);
        int U = m;
        bool rowdup = false;
        constexpr int kRowsPerPass = kIsFloat ? 4 : 8;   // 8 (4) lanes fetch one fp32 (16-bit) row
        const int prow = kIsFloat ? qi : (lane >> 2);
        int tok_reg[kUC / kRowsPerPass];                 // identical rows: source row of X row prow + kRowsPerPass * k
        if (identical) {
            const int* ring32 = reinterpret_cast<const int*>(ring);
#pragma unroll
            for (int k = 0; k < kUC / kRowsPerPass; ++k) {
                const int r = prow + kRowsPerPass * k;
                tok_reg[k] = r < m ? ring32[2 * r] : 0;
            }
        } else {
            U = dedup_tile(ds, ring, lut, E, m, i0, n, MODE == 0, &rowdup, lane);
        }
        __syncwarp();                                    // the landing area is free again

        for (int g = 0; g < heads; ++g) {
            const long long bb = (long long)b * heads + g;
            const T* Xh = X + (bb * n) * kC;
            float2 acc[2][2];
            acc[0][0] = acc[0][1] = acc[1][0] = acc[1][1] = make_float2(0.f, 0.f);
            float oreg[kEPL];
#pragma unroll
            for (int k = 0; k < kEPL; ++k) oreg[k] = 0.f;
            const int nchunks = U > 0 ? (U + kUC - 1) / kUC : 1;
            for (int ch = 0; ch < nchunks; ++ch) {
                const int u0 = ch * kUC;
                const int Uc = max(0, min(kUC, U - u0));
                const int rows8 = (Uc + 7) & ~7;
                __syncwarp();
                // ---- neighbour rows: 8 lanes x 16 bytes per fp32 row (4 lanes per 16-bit row)
                if (kIsFloat) {
#pragma unroll
                    for (int k = 0; k < kUC / 4; ++k) {
                        const int r = qi + 4 * k;
                        if (r < rows8) {
                            int t = -1;
                            if (r < Uc) {
                                if (identical) t = tok_reg[k];
                                else {
                                    const unsigned short tt = uniq[u0 + r];
                                    t = tt == kSkip ? -1 : (int)tt;
                                }
                            }
                            float* dst = Xs + r * kC + ((k & 1) ? sw_odd : sw_even);
                            if (t >= 0) cp_async16_ca(dst, Xh + (long long)t * kC + ci * 4);
                            else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                    }
                } else {
                    const int pr = lane >> 2, pc = lane & 3;
#pragma unroll
                    for (int k = 0; k < kUC / 8; ++k) {
                        const int r = pr + 8 * k;
                        if (r < rows8) {
                            int t = -1;
                            if (r < Uc) {
                                if (identical) t = tok_reg[k];
                                else {
                                    const unsigned short tt = uniq[u0 + r];
                                    t = tt == kSkip ? -1 : (int)tt;
                                }
                            }
                            T* dst = Xraw + r * kC + pc * kPer;
                            if (t >= 0) cp_async16_ca(dst, Xh + (long long)t * kC + pc * kPer);
                            else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                    }
                }
                cp_async_commit();

                if (MODE == 0) {
                    // ---- weight tile -> Wd, every weight twice, while the rows are on their way
                    const T* Wt = A + (bb * n + i0) * m;
                    if (identical) {
#pragma unroll
                        for (int k = 0; k < 3; ++k)
                            if (lane + 32 * k < kT * m4) {
                                const float4 w = ld4(Wt + wq[k] * m + wc[k] * 4);
                                float* dd = Wd + wq[k] * kWLD2 + wc[k] * 8;
                                *reinterpret_cast<float4*>(dd) = make_float4(w.x, w.x, w.y, w.y);
                                *reinterpret_cast<float4*>(dd + 4) = make_float4(w.z, w.z, w.w, w.w);
                            }
                    } else {
                        for (int z = lane; z < kT * kWLD2 / 4; z += 32)
                            reinterpret_cast<float4*>(Wd)[z] = make_float4(0.f, 0.f, 0.f, 0.f);
                        __syncwarp();
                        if (!rowdup) {
#pragma unroll
                            for (int k = 0; k < kEPL; ++k) {
                                const int x = lane + 32 * k;
                                if (x < E) {
                                    const unsigned short sl = lut[x];
                                    const int rel = (int)sl - u0;
                                    if (sl != kSkip && rel >= 0 && rel < Uc) {
                                        const float w = Elem<T>::up(Wt[x]);
                                        const int q = (int)((qpack >> (3 * k)) & 7ull);
                                        *reinterpret_cast<float2*>(Wd + q * kWLD2 + 2 * rel) = make_float2(w, w);
                                    }
                                }
                            }
                        } else if (lane < kT) {
                            // some row repeats a neighbour: one lane per row adds the weights in column order
                            for (int j = 0; j < m; ++j) {
                                const unsigned short sl = lut[lane * m + j];
                                const int rel = (int)sl - u0;
                                if (sl != kSkip && rel >= 0 && rel < Uc) {
                                    float2* cell = reinterpret_cast<float2*>(Wd + lane * kWLD2 + 2 * rel);
                                    const float w = cell->x + Elem<T>::up(Wt[lane * m + j]);
                                    *cell = make_float2(w, w);
                                }
                            }
                        }
                    }
                } else if (ch == 0) {
                    // ---- Y tile -> Ys (fp32, row stride kYLD)
                    const T* Yt = A + (bb * n + i0) * kC;
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const int z = lane + 32 * k;
                        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (i0 + (z >> 3) < n) v = ld4(Yt + z * 4);
                        *reinterpret_cast<float4*>(Ys + (z >> 3) * kYLD + (z & 7) * 4) = v;
                    }
                }
                cp_async_wait<0>();
                __syncwarp();
                if (!kIsFloat) {
                    // 16-bit rows -> fp32, swizzled
#pragma unroll
                    for (int k = 0; k < kUC / 4; ++k) {
                        const int r = qi + 4 * k;
                        if (r < rows8) st4(Xs + r * kC + ((k & 1) ? sw_odd : sw_even), ld4(Xraw + r * kC + ci * 4));
                    }
                    __syncwarp();
                }

                if (MODE == 0) {
                    sum_product(Wd, Xs, rows8, qi, swz, acc);
                } else {
                    dot_product(Ys, Xs, Sb, (Uc + 7) >> 3, qi, ci);
                    __syncwarp();
                    T* Ot = out + (bb * n + i0) * m;
                    if (identical) {
#pragma unroll
                        for (int k = 0; k < 3; ++k)
                            if (lane + 32 * k < kT * m4)
                                st4(Ot + wq[k] * m + wc[k] * 4, ld4(Sb + wq[k] * kWLD + wc[k] * 4));
                    } else {
#pragma unroll
                        for (int k = 0; k < kEPL; ++k) {
                            const int x = lane + 32 * k;
                            if (x < E) {
                                const unsigned short sl = lut[x];
                                const int rel = (int)sl - u0;
                                const int q = (int)((qpack >> (3 * k)) & 7ull);
                                if (sl != kSkip && rel >= 0 && rel < Uc) oreg[k] = Sb[q * kWLD + rel];
                            }
                        }
                        if (ch == nchunks - 1) {
#pragma unroll
                            for (int k = 0; k < kEPL; ++k) {
                                const int x = lane + 32 * k;
                                const int q = (int)((qpack >> (3 * k)) & 7ull);
                                if (x < E && i0 + q < n) Ot[x] = Elem<T>::down(oreg[k]);
                            }
                        }
                    }
                }
            }
            if (MODE == 0) {
#pragma unroll
                for (int a = 0; a < 2; ++a) {
                    const int i = i0 + 2 * qi + a;
                    if (i < n)
                        st4(out + (bb * n + i) * kC + ci * 4,
                            make_float4(acc[a][0].x, acc[a][0].y, acc[a][1].x, acc[a][1].y));
                }
            }
        }
    }
}

// ----------------------------------------------------------------------------- host side
bool gather_supported(int dtype, std::initializer_list<const void*> ptrs, int n, int m, int c) {
    if (c != kC || m < 1 || m > kMmax || n < 1 || n > 65000) return false;
    if (dtype != CLUSTEN_F32 && dtype != CLUSTEN_F16 && dtype != CLUSTEN_BF16) return false;
    for (const void* p : ptrs)
        if (reinterpret_cast<uintptr_t>(p) % 16 != 0) return false;
    return true;
}

template <typename T, int MODE>
int gather_tiles_t(const char* label, const void* A, const void* X, const int64_t* idx, void* out, int b, int h,
                   int n, int m, cudaStream_t s) {
    const int tiles = (n + kT - 1) / kT;
    const size_t smem = size_t(kWarps) * WarpSmem<T, MODE>::kTotal;
    auto kernel = gather_tiles_kernel<T, MODE>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return CLUSTEN_ERR_CUDA;
    }
    // one resident wave of CTAs; every warp strides over the (batch, tile) pairs
    const int per_sm = (int)((227 * 1024) / (smem + 1024));
    long long grid = (long long)sm_count() * (per_sm > 0 ? per_sm : 1);
    const long long need = ((long long)b * tiles + kWarps - 1) / kWarps;
    if (grid > need) grid = need;
    ScopedKernelTimer timer(label, s);
    kernel<<<(int)grid, 32 * kWarps, smem, s>>>((const T*)A, (const T*)X, idx, (T*)out, b, h, n, m, tiles);
    note_launch();
    return check_launch();
}

}  // namespace

int read_device_status(int* status, bool clear) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        return CLUSTEN_ERR_CUDA;
    }
    if (clear && v != 0) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)) != cudaSuccess) {
            cudaGetLastError();
            return CLUSTEN_ERR_CUDA;
        }
    }
    *status = v;
    return CLUSTEN_OK;
}

bool tiled_sum_supported(int dtype, const void* W, const void* X, const void* out, int n, int m, int c) {
    return gather_supported(dtype, {W, X, out}, n, m, c);
}
int launch_tiled_sum(const char* label, int dtype, const void* W, const void* X, const int64_t* idx, void* out,
                     int b, int h, int n, int m, cudaStream_t s) {
    switch (dtype) {
        case CLUSTEN_F32: return gather_tiles_t<float, 0>(label, W, X, idx, out, b, h, n, m, s);
        case CLUSTEN_F16: return gather_tiles_t<__half, 0>(label, W, X, idx, out, b, h, n, m, s);
        case CLUSTEN_BF16: return gather_tiles_t<__nv_bfloat16, 0>(label, W, X, idx, out, b, h, n, m, s);
        default: return CLUSTEN_ERR_DTYPE;
    }
}

bool tiled_dot_supported(int dtype, const void* Y, const void* X, const void* out, int n, int m, int c) {
    return gather_supported(dtype, {Y, X, out}, n, m, c);
}
int launch_tiled_dot(const char* label, int dtype, const void* X, const void* Y, const int64_t* idx, void* out,
                     int b, int h, int n, int m, cudaStream_t s) {
    switch (dtype) {
        case CLUSTEN_F32: return gather_tiles_t<float, 1>(label, Y, X, idx, out, b, h, n, m, s);
        case CLUSTEN_F16: return gather_tiles_t<__half, 1>(label, Y, X, idx, out, b, h, n, m, s);
        case CLUSTEN_BF16: return gather_tiles_t<__nv_bfloat16, 1>(label, Y, X, idx, out, b, h, n, m, s);
        default: return CLUSTEN_ERR_DTYPE;
    }
}

}  // namespace clusten
