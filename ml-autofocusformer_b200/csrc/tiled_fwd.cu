// Pipelined tiled kernels for the gather side of QK / AV (head_dim 32, m <= 48):
//
//   tiled_sum   out[i,:] = sum_j W[i,j] * X[idx[i,j],:]     AV forward, d_query
//   tiled_dot   out[i,j] = <X[idx[i,j],:], Y[i,:]>          QK forward, d_attn
//
// A CTA walks over consecutive tiles of 8 rows (one AutoFocusFormer cluster) of one batch
// element; warp w serves heads w, w+W, ...  The neighbour indices of a tile are read ONCE for
// all heads, two tiles ahead, straight into a shared-memory ring with cp.async.  When the 8
// rows of a tile are identical (the tokens of a cluster share their neighbourhood) the slot of
// a neighbour is simply its column; otherwise the tile's indices are de-duplicated with a
// bitmap over token ids (slots ascend with the token id).  Every head then stages each distinct
// neighbour row once (cp.async, 16-byte chunks, XOR-swizzled) and serves the 8 rows of the
// tile from shared memory with a register-tiled product; for identical rows the operands of
// the next (tile, head) are in flight while the current one is multiplied.
//
// The reference gives each output element a thread that re-gathers its neighbour rows from L2
// (clusten/src/clustenav_cuda_kernel.cu:18-50, clustenqk_cuda_kernel.cu:18-49).
#include <limits.h>
#include <type_traits>

#include "tiled.cuh"

namespace clusten {

namespace {

constexpr int kT = 8;            // rows per tile
constexpr int kC = 32;           // channels per head
constexpr int kMmax = 48;        // neighbours per row handled here
constexpr int kE = kT * kMmax;   // edges per tile
constexpr int kUC = 48;          // distinct neighbour rows staged at a time
constexpr int kWLD = 52;         // row stride (floats) of the score tile
constexpr int kWLD2 = 100;       // row stride (floats) of the weight tile, every weight stored twice
constexpr int kYLD = 36;         // row stride (floats) of the staged Y tile
constexpr int kRing = 3;         // index tiles in flight
constexpr int kBMW = 256;        // bitmap words: token ids of a tile may span 8192
constexpr int kMaxWarps = 4;
constexpr int kEPL = kE / 32;    // edges per lane
constexpr unsigned kFull = 0xffffffffu;
constexpr unsigned short kSkip = 0xffffu;
constexpr unsigned short kRowDup = 0x8000u;

struct Smem {
    long long ring[kRing][kE];          // raw int64 neighbour indices of up to three tiles
    unsigned short tok[kE];             // general path: source row of each edge, kSkip = none
    unsigned short slot[kE];            // general path: edge -> slot (| kRowDup), kSkip = contributes nothing
    unsigned short uniq[kE];            // general path: slot -> source row
    unsigned bm[kBMW];
    unsigned short pre[kBMW];
    unsigned rowbm[kMaxWarps][kE / 32];
    int misc[8];                        // [0]=U [1]=min [2]=max
    int warp_tot[kMaxWarps];
};

// per warp: two buffers of neighbour rows, and
//   tiled_sum: one weight tile [8][kWLD2] (each weight twice, for the two-wide FMA)
//   tiled_dot: two Y tiles [8][kYLD] and one score tile [8][kWLD]
constexpr int kXFloats = kUC * kC;                  // 1536
constexpr int kWFloats = kT * kWLD2;                // 800
constexpr int kYFloats = kT * kYLD;                 // 288
__host__ __device__ constexpr int warp_floats(int mode) {
    return 2 * kXFloats + (mode == 0 ? kWFloats : 2 * kYFloats + kT * kWLD);
}

constexpr size_t kSmemHead = (sizeof(Smem) + 15) & ~size_t(15);
inline size_t smem_bytes(int warps, int mode) {
    return kSmemHead + size_t(warps) * warp_floats(mode) * sizeof(float);
}

// ----------------------------------------------------------------------------- small helpers
__device__ __forceinline__ void cp_async16_ca(void* smem_dst, const void* gsrc) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gsrc));
}
__device__ __forceinline__ void cp_async16_cg(void* smem_dst, const void* gsrc) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gsrc));
}
__device__ __forceinline__ void cp_async8_ca(void* smem_dst, const void* gsrc) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(d), "l"(gsrc));
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

// Sb[2qi+a][8k+ui] = <Ys[2qi+a][:], Xs[8k+ui][:]> for k < kmax; packed two-wide FMAs over channel pairs
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

// ----------------------------------------------------------------------------- general path: de-duplication
// ring tile -> tok / slot / uniq.  All threads of the CTA.  Returns U.
__device__ int dedup_tile(Smem* sm, const long long* __restrict__ ring, int E, int m, int i0, int n_rows,
                          int n_src) {
    const int tid = threadIdx.x, nth = blockDim.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        sm->misc[1] = INT_MAX;
        sm->misc[2] = -1;
    }
    __syncthreads();
    int lo = INT_MAX, hi = -1;
    for (int x = tid; x < E; x += nth) {
        const long long v = ring[x];
        const int q = x / m;
        unsigned short t = kSkip;
        if (i0 + q < n_rows && v >= 0 && v < n_src) {
            t = (unsigned short)v;
            lo = min(lo, (int)v);
            hi = max(hi, (int)v);
        }
        sm->tok[x] = t;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        lo = min(lo, __shfl_xor_sync(kFull, lo, o));
        hi = max(hi, __shfl_xor_sync(kFull, hi, o));
    }
    if (lane == 0) {
        atomicMin(&sm->misc[1], lo);
        atomicMax(&sm->misc[2], hi);
    }
    __syncthreads();
    lo = sm->misc[1];
    hi = sm->misc[2];
    if (hi < 0) {
        for (int x = tid; x < E; x += nth) sm->slot[x] = kSkip;
        __syncthreads();
        return 0;
    }
    const int w0 = lo >> 5;
    const int words = (hi >> 5) - w0 + 1;
    if (words > kBMW) {                      // ids too spread out: one slot per edge
        for (int x = tid; x < E; x += nth) {
            const unsigned short t = sm->tok[x];
            sm->slot[x] = t != kSkip ? (unsigned short)x : kSkip;
            sm->uniq[x] = t;
        }
        __syncthreads();
        return E;
    }
    for (int w = tid; w < words; w += nth) sm->bm[w] = 0u;
    __syncthreads();
    for (int x = tid; x < E; x += nth) {
        const unsigned short t = sm->tok[x];
        if (t != kSkip) atomicOr(&sm->bm[(t >> 5) - w0], 1u << (t & 31));
    }
    __syncthreads();
    {
        const int per = (words + nth - 1) / nth;
        const int a = min(tid * per, words), b = min(a + per, words);
        int local = 0;
        for (int w = a; w < b; ++w) local += __popc(sm->bm[w]);
        int incl = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int y = __shfl_up_sync(kFull, incl, o);
            if (lane >= o) incl += y;
        }
        if (lane == 31) sm->warp_tot[warp] = incl;
        __syncthreads();
        int run = incl - local;
        for (int w = 0; w < warp; ++w) run += sm->warp_tot[w];
        for (int w = a; w < b; ++w) {
            sm->pre[w] = (unsigned short)run;
            run += __popc(sm->bm[w]);
        }
        if (tid == nth - 1) sm->misc[0] = run;
    }
    __syncthreads();
    for (int x = tid; x < E; x += nth) {
        const unsigned short t = sm->tok[x];
        if (t != kSkip) {
            const int w = (t >> 5) - w0;
            const int s = sm->pre[w] + __popc(sm->bm[w] & ((1u << (t & 31)) - 1u));
            sm->slot[x] = (unsigned short)s;
            sm->uniq[s] = t;
        } else {
            sm->slot[x] = kSkip;
        }
    }
    __syncthreads();
    return sm->misc[0];
}

// A row may name the same neighbour several times.  Detection: each warp ORs the slots of one row
// at a time into a small bitmap.  Only if some row has a repeat is the exact bookkeeping done: the
// first occurrence keeps the slot and is flagged kRowDup (its weight becomes the sum of the row's
// occurrences in column order), later occurrences are skipped.
__device__ void resolve_row_duplicates(Smem* sm, int E, int m, int U) {
    const int tid = threadIdx.x, nth = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarps = nth >> 5;
    unsigned* rb = sm->rowbm[warp];
    const int words = (U + 31) >> 5;
    int seen = 0;
    for (int q = warp; q < kT; q += nwarps) {
        if (lane < words) rb[lane] = 0u;
        __syncwarp();
        for (int jj = lane; jj < m; jj += 32) {
            const unsigned short s = sm->slot[q * m + jj];
            if (s != kSkip) {
                const unsigned bit = 1u << (s & 31);
                if (atomicOr(&rb[s >> 5], bit) & bit) seen = 1;
            }
        }
        __syncwarp();
    }
    if (!__syncthreads_or(seen)) return;
    for (int x = tid; x < E; x += nth) {
        unsigned short s = sm->slot[x];
        if (s == kSkip) continue;
        const int q = x / m, jj = x - q * m;
        const unsigned short t = sm->tok[x];
        bool first = true, later = false;
        for (int j2 = 0; j2 < m; ++j2) {
            if (j2 != jj && sm->tok[q * m + j2] == t) {
                if (j2 < jj) first = false;
                else later = true;
            }
        }
        sm->slot[x] = !first ? kSkip : (later ? (unsigned short)(s | kRowDup) : s);
    }
    __syncthreads();
}

// stage rows uniq[u0..u0+rows) of one head into Xs (rows beyond U zero-filled); one warp, synchronous
template <typename T>
__device__ __forceinline__ void stage_rows_sync(float* __restrict__ Xs, const T* __restrict__ Xh,
                                                const unsigned short* __restrict__ uniq, int u0, int U,
                                                int rows4, int lane) {
    const int chunk = lane & 7;
#pragma unroll 4
    for (int r = lane >> 3; r < rows4; r += 4) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (u0 + r < U) {
            const unsigned short t = uniq[u0 + r];
            if (t != kSkip) v = ld4(Xh + (long long)t * kC + chunk * 4);
        }
        st4(Xs + r * kC + ((chunk ^ (r & 7)) << 2), v);
    }
}

// ----------------------------------------------------------------------------- the kernel
// MODE 0: tiled_sum (A = W [bb, n, m]),  MODE 1: tiled_dot (A = Y [bb, n, 32]); X = [bb, n, 32]
template <typename T, int MODE>
__global__ void __launch_bounds__(32 * kMaxWarps, 4)
tiled_gather_kernel(const T* __restrict__ A, const T* __restrict__ X, const int64_t* __restrict__ idx,
                    T* __restrict__ out, int heads, int n, int m, int tiles, int tiles_per_cta) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Smem* sm = reinterpret_cast<Smem*>(smem_raw);
    const int tid = threadIdx.x, nth = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, nwarps = nth >> 5;
    const int qi = lane >> 3, ci = lane & 7;
    float* wbase = reinterpret_cast<float*>(smem_raw + kSmemHead) + size_t(warp) * warp_floats(MODE);
    float* const Xb0 = wbase;
    float* const Xb1 = wbase + kXFloats;
    float* const Wd = wbase + 2 * kXFloats;                 // MODE 0: weight tile
    float* const Yb0 = wbase + 2 * kXFloats;                // MODE 1: Y tiles and score tile
    float* const Yb1 = Yb0 + kYFloats;
    float* const Sb = Yb1 + kYFloats;
    constexpr bool kAsync = std::is_same<T, float>::value;

    const int groups = (tiles + tiles_per_cta - 1) / tiles_per_cta;
    const int b = blockIdx.x / groups;
    const int tile_begin = (blockIdx.x - b * groups) * tiles_per_cta;
    const int tile_end = min(tile_begin + tiles_per_cta, tiles);
    const int64_t* idx_b = idx + (long long)b * n * m;
    const int E = kT * m;
    const int m4 = m >> 2;
    const bool vec_ok = (m & 7) == 0;          // rows move in 16-byte pieces and the product runs 8 neighbours at a time
    const bool idx16 = (E & 1) == 0 && (reinterpret_cast<uintptr_t>(idx_b) & 15) == 0;

    int swz[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) swz[k] = (ci ^ k) << 2;
    const int sw_even = (ci ^ qi) << 2, sw_odd = sw_even ^ 16;   // swizzle of row qi + 4k, k even / odd
    // weight / score chunk z = lane + 32k of a tile -> (row, 16-byte chunk)
    int wq[3], wc[3];
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        const int z = lane + 32 * k;
        const int d = m4 > 0 ? m4 : 1;
        wq[k] = z / d;
        wc[k] = z - wq[k] * d;
    }
    const int col0 = (2 * tid) % m, col_step = (2 * nth) % m;   // column of entry pair 2 * (tid + k * nth)

    // ---- raw indices of `tile` -> ring (all threads; always commits one group)
    auto issue_index = [&](int tile) {
        if (tile < tile_end) {
            long long* dst = sm->ring[tile % kRing];
            const int64_t* src = idx_b + (long long)tile * E;
            if (tile * kT + kT <= n && idx16) {
                for (int x = 2 * tid; x < E; x += 2 * nth) cp_async16_ca(dst + x, src + x);
            } else {
                const int valid = min(kT, n - tile * kT) * m;
                for (int x = tid; x < E; x += nth) {
                    if (x < valid) cp_async8_ca(dst + x, src + x);
                    else dst[x] = -1;
                }
            }
        }
        cp_async_commit();
    };

    // ---- are the 8 rows of `tile` identical, in range, and the tile complete?  (all threads)
    auto rows_identical = [&](int tile) -> bool {
        const int4* r = reinterpret_cast<const int4*>(sm->ring[tile % kRing]);   // {lo, hi, lo, hi}
        int same = (tile * kT + kT <= n && vec_ok) ? 1 : 0;
        int col = col0;
        for (int x = tid; 2 * x < E; x += nth) {
            const int4 v = r[x];
            const int4 ref = r[col >> 1];
            if (v.x != ref.x || v.z != ref.z || (v.y | v.w) != 0 || (unsigned)v.x >= (unsigned)n ||
                (unsigned)v.z >= (unsigned)n)
                same = 0;
            col += col_step;
            if (col >= m) col -= m;
        }
        return __syncthreads_and(same) != 0;
    };

    // ---- neighbour rows of (tile, head g), identical-rows case: row r of the tile's first index row
    auto issue_rows = [&](int tile, int g, float* Xs) {
        const int* row0 = reinterpret_cast<const int*>(sm->ring[tile % kRing]);
        const T* Xh = X + (((long long)b * heads + g) * n) * kC + ci * 4;
        float* dst = Xs + qi * kC;
#pragma unroll
        for (int k = 0; k < kUC / 4; ++k) {
            const int r = qi + 4 * k;
            if (r < m) cp_async16_ca(dst + 4 * k * kC + ((k & 1) ? sw_odd : sw_even), Xh + (long long)row0[2 * r] * kC);
        }
    };
    auto issue_y = [&](int tile, int g, float* Ys) {
        const T* Yt = A + (((long long)b * heads + g) * n + tile * kT) * kC;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int z = lane + 32 * k;
            cp_async16_cg(Ys + (z >> 3) * kYLD + (z & 7) * 4, Yt + z * 4);
        }
    };
    // weight tile: global -> registers (early) -> shared, every weight twice (late)
    auto load_w = [&](int tile, int g, float4 (&wr)[3]) {
        const T* Wt = A + (((long long)b * heads + g) * n + tile * kT) * m;
#pragma unroll
        for (int k = 0; k < 3; ++k)
            if (lane + 32 * k < kT * m4) wr[k] = ld4(Wt + wq[k] * m + wc[k] * 4);
    };
    auto store_w = [&](const float4 (&wr)[3]) {
#pragma unroll
        for (int k = 0; k < 3; ++k)
            if (lane + 32 * k < kT * m4) {
                float* d = Wd + wq[k] * kWLD2 + wc[k] * 8;
                *reinterpret_cast<float4*>(d) = make_float4(wr[k].x, wr[k].x, wr[k].y, wr[k].y);
                *reinterpret_cast<float4*>(d + 4) = make_float4(wr[k].z, wr[k].z, wr[k].w, wr[k].w);
            }
    };

    // ------------------------------------------------------------------ prologue
    issue_index(tile_begin);
    issue_index(tile_begin + 1);
    cp_async_wait<1>();
    __syncthreads();
    bool cur_same = rows_identical(tile_begin);
    int buf = 0;
    bool have_prefetch = false;            // operands of this warp's next task are under way
    float4 wnext[3];
    wnext[0] = wnext[1] = wnext[2] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (cur_same && kAsync) {
        issue_rows(tile_begin, warp, Xb0);
        if (MODE == 0) {
            load_w(tile_begin, warp, wnext);
            store_w(wnext);
        } else {
            issue_y(tile_begin, warp, Yb0);
        }
        have_prefetch = true;
    }
    cp_async_commit();

    for (int tile = tile_begin; tile < tile_end; ++tile) {
        const int i0 = tile * kT;
        // ---- look ahead: indices of tile+2 start moving, tile+1 is classified
        issue_index(tile + 2);
        cp_async_wait<1>();                // everything but the newest group has landed
        __syncthreads();
        bool next_same = false;
        if (tile + 1 < tile_end) next_same = rows_identical(tile + 1);
        if (tid * 16 < E && tile + 4 < tile_end) prefetch_l2(idx_b + (long long)(tile + 4) * E + tid * 16);

        int U = m;
        if (!cur_same) {
            U = dedup_tile(sm, sm->ring[tile % kRing], E, m, i0, n, n);
            if (MODE == 0 && U > 0 && U < E) resolve_row_duplicates(sm, E, m, U);
        }

        bool first_task = true;
        for (int g = warp; g < heads; g += nwarps) {
            const long long bb = (long long)b * heads + g;
            const T* Xh = X + (bb * n) * kC;
            float* Xs = buf ? Xb1 : Xb0;
            float* Xn = buf ? Xb0 : Xb1;
            float* Ys = buf ? Yb1 : Yb0;
            float* Yn = buf ? Yb0 : Yb1;
            // ---- start moving the operands of the task after this one
            const bool had = have_prefetch;
            have_prefetch = false;
            int nt = -1, ng = 0;
            if (kAsync) {
                if (g + nwarps < heads) {
                    if (cur_same) { nt = tile; ng = g + nwarps; }
                } else if (next_same) {
                    nt = tile + 1; ng = warp;
                }
                if (nt >= 0) {
                    issue_rows(nt, ng, Xn);
                    if (MODE == 0) load_w(nt, ng, wnext);
                    else issue_y(nt, ng, Yn);
                    have_prefetch = true;
                }
            }
            cp_async_commit();

            if (cur_same) {
                // ================= identical rows: slot = column
                if (kAsync) {
                    if (!had) {                         // nothing was under way for this task
                        float4 wnow[3];
                        issue_rows(tile, g, Xs);
                        if (MODE == 0) {
                            load_w(tile, g, wnow);
                            __syncwarp();
                            store_w(wnow);
                        } else {
                            issue_y(tile, g, Ys);
                        }
                        cp_async_commit();
                        cp_async_wait<0>();
                    } else if (first_task) {
                        cp_async_wait<2>();             // may still fly: indices two tiles ahead, next task's operands
                    } else {
                        cp_async_wait<1>();
                    }
                } else {
                    __syncwarp();
                    const int* row0 = reinterpret_cast<const int*>(sm->ring[tile % kRing]);
#pragma unroll
                    for (int k = 0; k < kUC / 4; ++k) {
                        const int r = qi + 4 * k;
                        if (r < m)
                            st4(Xs + r * kC + ((k & 1) ? sw_odd : sw_even),
                                ld4(Xh + (long long)row0[2 * r] * kC + ci * 4));
                    }
                    if (MODE == 0) {
                        float4 wnow[3];
                        load_w(tile, g, wnow);
                        store_w(wnow);
                    } else {
                        const T* Yt = A + (bb * n + i0) * kC;
#pragma unroll
                        for (int k = 0; k < 2; ++k) {
                            const int z = lane + 32 * k;
                            st4(Ys + (z >> 3) * kYLD + (z & 7) * 4, ld4(Yt + z * 4));
                        }
                    }
                }
                __syncwarp();
                if (MODE == 0) {
                    float2 acc[2][2];
                    acc[0][0] = acc[0][1] = acc[1][0] = acc[1][1] = make_float2(0.f, 0.f);
                    sum_product(Wd, Xs, m, qi, swz, acc);
#pragma unroll
                    for (int a = 0; a < 2; ++a)
                        st4(out + (bb * n + i0 + 2 * qi + a) * kC + ci * 4,
                            make_float4(acc[a][0].x, acc[a][0].y, acc[a][1].x, acc[a][1].y));
                    __syncwarp();                              // the weight tile is free again
                    if (have_prefetch) store_w(wnext);
                } else {
                    dot_product(Ys, Xs, Sb, (m + 7) >> 3, qi, ci);
                    __syncwarp();
                    T* Ot = out + (bb * n + i0) * m;
#pragma unroll
                    for (int k = 0; k < 3; ++k)
                        if (lane + 32 * k < kT * m4)
                            st4(Ot + wq[k] * m + wc[k] * 4, ld4(Sb + wq[k] * kWLD + wc[k] * 4));
                    __syncwarp();
                }
            } else {
                // ================= general rows: dense [8 x U] weights over de-duplicated neighbours
                if (MODE == 0) {
                    const T* Wh = A + (bb * n) * m;
                    float wreg[kEPL];
#pragma unroll
                    for (int k = 0; k < kEPL; ++k) {
                        const int x = lane + 32 * k;
                        float w = 0.f;
                        if (x < E) {
                            const unsigned short s = sm->slot[x];
                            if (s != kSkip) {
                                const int q = x / m, jj = x - q * m;
                                const T* wrow = Wh + (long long)(i0 + q) * m;
                                w = Elem<T>::up(wrow[jj]);
                                if (s & kRowDup) {
                                    const unsigned short t = sm->tok[x];
                                    for (int j2 = jj + 1; j2 < m; ++j2)
                                        if (sm->tok[q * m + j2] == t) w += Elem<T>::up(wrow[j2]);
                                }
                            }
                        }
                        wreg[k] = w;
                    }
                    float2 acc[2][2];
                    acc[0][0] = acc[0][1] = acc[1][0] = acc[1][1] = make_float2(0.f, 0.f);
                    for (int u0 = 0; u0 < U; u0 += kUC) {
                        const int Uc = min(kUC, U - u0);
                        const int rows8 = (Uc + 7) & ~7;
                        __syncwarp();
                        stage_rows_sync<T>(Xs, Xh, sm->uniq, u0, U, rows8, lane);
                        for (int z = lane; z < kWFloats / 4; z += 32)
                            reinterpret_cast<float4*>(Wd)[z] = make_float4(0.f, 0.f, 0.f, 0.f);
                        __syncwarp();
#pragma unroll
                        for (int k = 0; k < kEPL; ++k) {
                            const int x = lane + 32 * k;
                            if (x < E) {
                                const unsigned short s = sm->slot[x];
                                const int sl = (s & 0x7fff) - u0;
                                if (s != kSkip && sl >= 0 && sl < Uc)
                                    *reinterpret_cast<float2*>(Wd + (x / m) * kWLD2 + 2 * sl) =
                                        make_float2(wreg[k], wreg[k]);
                            }
                        }
                        __syncwarp();
                        sum_product(Wd, Xs, rows8, qi, swz, acc);
                    }
#pragma unroll
                    for (int a = 0; a < 2; ++a) {
                        const int i = i0 + 2 * qi + a;
                        if (i < n)
                            st4(out + (bb * n + i) * kC + ci * 4,
                                make_float4(acc[a][0].x, acc[a][0].y, acc[a][1].x, acc[a][1].y));
                    }
                    __syncwarp();
                    if (have_prefetch) store_w(wnext);
                } else {
                    const T* Yh = A + (bb * n) * kC;
                    T* Oh = out + (bb * n) * m;
                    __syncwarp();
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const int z = lane + 32 * k;
                        const int q = z >> 3;
                        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (i0 + q < n) v = ld4(Yh + (long long)(i0 + q) * kC + (z & 7) * 4);
                        st4(Ys + q * kYLD + (z & 7) * 4, v);
                    }
                    float oreg[kEPL];
#pragma unroll
                    for (int k = 0; k < kEPL; ++k) oreg[k] = 0.f;
                    for (int u0 = 0; u0 < U; u0 += kUC) {
                        const int Uc = min(kUC, U - u0);
                        __syncwarp();
                        stage_rows_sync<T>(Xs, Xh, sm->uniq, u0, U, (Uc + 3) & ~3, lane);
                        __syncwarp();
                        dot_product(Ys, Xs, Sb, (Uc + 7) >> 3, qi, ci);
                        __syncwarp();
#pragma unroll
                        for (int k = 0; k < kEPL; ++k) {
                            const int x = lane + 32 * k;
                            if (x < E) {
                                const unsigned short s = sm->slot[x];
                                const int sl = (int)s - u0;
                                if (s != kSkip && sl >= 0 && sl < Uc) oreg[k] = Sb[(x / m) * kWLD + sl];
                            }
                        }
                    }
#pragma unroll
                    for (int k = 0; k < kEPL; ++k) {
                        const int x = lane + 32 * k;
                        const int q = x / m;
                        if (x < E && i0 + q < n) Oh[(long long)(i0 + q) * m + (x - q * m)] = Elem<T>::down(oreg[k]);
                    }
                }
            }
            buf ^= 1;
            first_task = false;
        }
        cur_same = next_same;
        __syncthreads();
    }
    cp_async_wait<0>();
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
int tiled_gather_t(const char* label, const void* A, const void* X, const int64_t* idx, void* out, int b, int h,
                   int n, int m, cudaStream_t s) {
    const int warps = h < kMaxWarps ? h : kMaxWarps;
    const int tiles = (n + kT - 1) / kT;
    // enough CTAs to fill the machine a few times over, consecutive tiles per CTA for the pipeline
    int tpc = 8;
    while (tpc > 1 && (long long)b * ((tiles + tpc - 1) / tpc) < (long long)sm_count() * 8) tpc >>= 1;
    const int grid = b * ((tiles + tpc - 1) / tpc);
    const size_t smem = smem_bytes(warps, MODE);
    auto kernel = tiled_gather_kernel<T, MODE>;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return CLUSTEN_ERR_CUDA;
    }
    ScopedKernelTimer timer(label, s);
    kernel<<<grid, 32 * warps, smem, s>>>((const T*)A, (const T*)X, idx, (T*)out, h, n, m, tiles, tpc);
    note_launch();
    return check_launch();
}

}  // namespace

bool tiled_sum_supported(int dtype, const void* W, const void* X, const void* out, int n, int m, int c) {
    return gather_supported(dtype, {W, X, out}, n, m, c);
}
int launch_tiled_sum(const char* label, int dtype, const void* W, const void* X, const int64_t* idx, void* out,
                     int b, int h, int n, int m, cudaStream_t s) {
    switch (dtype) {
        case CLUSTEN_F32: return tiled_gather_t<float, 0>(label, W, X, idx, out, b, h, n, m, s);
        case CLUSTEN_F16: return tiled_gather_t<__half, 0>(label, W, X, idx, out, b, h, n, m, s);
        case CLUSTEN_BF16: return tiled_gather_t<__nv_bfloat16, 0>(label, W, X, idx, out, b, h, n, m, s);
        default: return CLUSTEN_ERR_DTYPE;
    }
}

bool tiled_dot_supported(int dtype, const void* Y, const void* X, const void* out, int n, int m, int c) {
    return gather_supported(dtype, {Y, X, out}, n, m, c);
}
int launch_tiled_dot(const char* label, int dtype, const void* X, const void* Y, const int64_t* idx, void* out,
                     int b, int h, int n, int m, cudaStream_t s) {
    switch (dtype) {
        case CLUSTEN_F32: return tiled_gather_t<float, 1>(label, Y, X, idx, out, b, h, n, m, s);
        case CLUSTEN_F16: return tiled_gather_t<__half, 1>(label, Y, X, idx, out, b, h, n, m, s);
        case CLUSTEN_BF16: return tiled_gather_t<__nv_bfloat16, 1>(label, Y, X, idx, out, b, h, n, m, s);
        default: return CLUSTEN_ERR_DTYPE;
    }
}

}  // namespace clusten
