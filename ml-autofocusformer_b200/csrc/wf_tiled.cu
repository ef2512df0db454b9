// Tiled CLUSTENWF kernels (gather side): feat_new = weights^T x gathered features, and d_weights.
//
//   wf_sum   out[b,i,k,:] = sum_j W[b,i,j,k] * F[b, idx[b,i,j], :]          (forward)
//   wf_dot   dW[b,i,j,k]  = <F[b, idx[b,i,j], :], dO[b,i,k,:]>              (d_weights)
//
// The merge centres arrive in no particular order (models/aff_transformer.py:320-336 of the reference
// picks them with an unsorted top-k), so consecutive rows of nbhd_idx share nothing.  A small pre-pass
// orders the rows of each batch element by their first neighbour (wf_order_kernel, bitonic sort in
// shared memory); a warp then takes 8 rows that are adjacent in that order -- spatial neighbours -- and,
// as in the attention kernels, de-duplicates their 8 x m indices (about 100 distinct rows instead of
// 384), stages every distinct feature row once, 32 rows x 64 channels at a time, and multiplies on the
// tensor cores against the dense [8 ic x 32] weights (forward) or the [8 ic x 64] gradient tile
// (d_weights).  The reference gathers every feature row ic times per output and neighbour
// (clusten/src/clustenwf_cuda_kernel.cu:41-47, :118-126).
#include "tile_core.cuh"

namespace clusten {
namespace {

// ----------------------------------------------------------------------------- row order
constexpr int kOrderMax = 4096;     // rows per batch element that the shared-memory sort handles
__global__ void __launch_bounds__(1024)
wf_order_kernel(const int64_t* __restrict__ idx, int* __restrict__ order, int n_out, int m) {
    __shared__ unsigned keys[kOrderMax];
    const int b = blockIdx.x, tid = threadIdx.x;
    int P = 1;
    while (P < n_out) P <<= 1;
    for (int i = tid; i < P; i += blockDim.x) {
        unsigned key = 0xffffffffu;
        if (i < n_out) {
            long long v = idx[((long long)b * n_out + i) * m];
            v = v < 0 ? 0 : (v > 65534 ? 65534 : v);
            key = ((unsigned)v << 16) | (unsigned)i;
        }
        keys[i] = key;
    }
    __syncthreads();
    for (int k = 2; k <= P; k <<= 1)
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = tid; i < P; i += blockDim.x) {
                const int l = i ^ j;
                if (l > i) {
                    const unsigned a = keys[i], c = keys[l];
                    const bool up = (i & k) == 0;
                    if ((a > c) == up) {
                        keys[i] = c;
                        keys[l] = a;
                    }
                }
            }
            __syncthreads();
        }
    for (int i = tid; i < n_out; i += blockDim.x) order[(long long)b * n_out + i] = (int)(keys[i] & 0xffffu);
}

// ----------------------------------------------------------------------------- tiles
constexpr int kUW = 32;             // distinct feature rows per stage
constexpr int kCG = 64;             // channels per stage
constexpr int kDL = 36;             // row stride (floats) of the dense weight tile and of the score tile, [32][kDL]
constexpr int kGL = 68;             // row stride (floats) of the gradient tile [32][kGL] and of the output tile [8][kGL]
constexpr int kRowsM = 32;          // (ic, row) pairs of a tile: M of the d_weights product, N of the forward one

struct WfParams {
    const void* W;        // wf_sum: weights [b, n_out, m, ic]
    const void* F;        // feat [b, n, c]
    const void* G;        // wf_dot: d_feat_new [b, n_out, ic, c]
    void* out;            // wf_sum: feat_new [b, n_out, ic, c];  wf_dot: d_weights [b, n_out, m, ic]
    const int64_t* idx;   // [b, n_out, m]
    const int* order;     // [b, n_out] or nullptr (storage order)
    int batch, n_out, n, m, c, tiles;
};

// per-warp shared memory
//   X    feature rows [32][64] fp32 (16-byte chunks XOR-swizzled with the row); before that the landing
//        area of the tile's indices and the token scratch; afterwards the output tile (wf_sum) or the
//        score tile (wf_dot)
//   Op   wf_sum: dense weights [8 ic][kDL];  wf_dot: gradient tile [8 ic][kGL];  bitmap scratch before that
//   lut  edge -> slot | tile row << 12,  uniq  slot -> feature row,  rows  the tile's 8 row numbers
template <int MODE> struct WfSmem {
    static constexpr int kX = kUW * kCG * 4;
    static constexpr int kOp = MODE == 0 ? kRowsM * kDL * 4 : kRowsM * kGL * 4;
    static constexpr int kLut = kE * 2;
    static constexpr int kRows = 32;
    static constexpr int kTotal = kX + kOp + 2 * kLut + kRows;
};
static_assert(kE * 8 + kE * 2 <= kUW * kCG * 4, "indices and token scratch must fit in the row buffer");
static_assert(kBMW * 4 + kBMW * 2 + (kE / 32) * 4 <= kRowsM * kDL * 4, "bitmap scratch must fit in Op");
static_assert(kRowsM * kDL * 4 <= kUW * kCG * 4 && kT * kGL * 4 <= kUW * kCG * 4, "score / output tile must fit in X");

#define WF_LDS(dst, addr, off) asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(dst) : "r"((addr) + (unsigned)(off)))

__device__ __forceinline__ unsigned fast_div_u(unsigned x, unsigned magic, unsigned shift) {
    return (__umulhi(magic, x) + x) >> shift;
}

template <bool SPLIT> __device__ __forceinline__ void wf_split(float x, unsigned& hi, unsigned& lo) {
    if (SPLIT) {
        split_tf32(x, hi, lo);
    } else {
        hi = __float_as_uint(x);
        lo = 0u;
    }
}
template <bool SPLIT>
__device__ __forceinline__ void wf_mma(float (&d)[4], const unsigned (&ah)[4], const unsigned (&al)[4],
                                       const unsigned (&bh)[2], const unsigned (&bl)[2]) {
    if (SPLIT) {
        mma_tf32(d, al, bh);
        mma_tf32(d, ah, bl);
    }
    mma_tf32(d, ah, bh);
}
// NM accumulators fed by the same B fragment, pass by pass: consecutive MMAs never share an accumulator
template <bool SPLIT, int NM>
__device__ __forceinline__ void wf_mma_row(float (&d)[NM][4], const unsigned (&ah)[NM][4], const unsigned (&al)[NM][4],
                                           const unsigned (&bh)[2], const unsigned (&bl)[2]) {
    if (SPLIT) {
#pragma unroll
        for (int mt = 0; mt < NM; ++mt) mma_tf32(d[mt], al[mt], bh);
#pragma unroll
        for (int mt = 0; mt < NM; ++mt) mma_tf32(d[mt], ah[mt], bl);
    }
#pragma unroll
    for (int mt = 0; mt < NM; ++mt) mma_tf32(d[mt], ah[mt], bh);
}

// 8 elements of T -> two float4
__device__ __forceinline__ void up8(const uint4 r, const __half*, float4& a, float4& b) {
    const float2 p0 = __half22float2(*reinterpret_cast<const __half2*>(&r.x));
    const float2 p1 = __half22float2(*reinterpret_cast<const __half2*>(&r.y));
    const float2 p2 = __half22float2(*reinterpret_cast<const __half2*>(&r.z));
    const float2 p3 = __half22float2(*reinterpret_cast<const __half2*>(&r.w));
    a = make_float4(p0.x, p0.y, p1.x, p1.y);
    b = make_float4(p2.x, p2.y, p3.x, p3.y);
}
__device__ __forceinline__ void up8(const uint4 r, const __nv_bfloat16*, float4& a, float4& b) {
    a = make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xffff0000u), __uint_as_float(r.y << 16),
                    __uint_as_float(r.y & 0xffff0000u));
    b = make_float4(__uint_as_float(r.z << 16), __uint_as_float(r.z & 0xffff0000u), __uint_as_float(r.w << 16),
                    __uint_as_float(r.w & 0xffff0000u));
}

// Stage rows8 rows of 64 channels into Xs (fp32, chunk c of row r at chunk ^ swz(r)); rows past n_rows
// are zero.  src(r) gives the global address of row r's 64 channels.  SWZ 0: (r & 3) << 1, 1: r & 7.
template <typename T, int SWZ, typename SrcFn>
__device__ __forceinline__ void stage_rows64(float* Xs, int rows8, int n_rows, int lane, SrcFn src) {
    if constexpr (std::is_same<T, float>::value) {
        const int rsub = lane >> 4, ch = lane & 15;
#pragma unroll 4
        for (int i = 0; i < kUW / 2; ++i) {
            const int r = 2 * i + rsub;
            if (r < rows8) {
                const int s = SWZ == 0 ? ((r & 3) << 1) : (r & 7);
                float* dst = Xs + r * kCG + ((ch ^ s) << 2);
                if (r < n_rows) cp_async16_cg(dst, src(r) + ch * 4);
                else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
    } else {
        const int rsub = lane >> 3, c8 = lane & 7;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            uint4 v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = 4 * (4 * half + i) + rsub;
                v[i] = make_uint4(0u, 0u, 0u, 0u);
                if (r < n_rows) v[i] = *reinterpret_cast<const uint4*>(src(r) + c8 * 8);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = 4 * (4 * half + i) + rsub;
                if (r < rows8) {
                    const int s = SWZ == 0 ? ((r & 3) << 1) : (r & 7);
                    float4 a, b;
                    up8(v[i], static_cast<const T*>(nullptr), a, b);
                    *reinterpret_cast<float4*>(Xs + r * kCG + (((2 * c8) ^ s) << 2)) = a;
                    *reinterpret_cast<float4*>(Xs + r * kCG + (((2 * c8 + 1) ^ s) << 2)) = b;
                }
            }
        }
    }
}

// 16-bit rows of 64 channels kept 16-bit: 128 bytes per row, 16-byte chunk c of row r at c ^ (r & 7)
// (conflict-free for ldmatrix with and without .trans)
constexpr int kDL16 = 40;           // row stride (elements) of the 16-bit dense weight tile
__device__ __forceinline__ int swz64(int r, int c) { return r * kCG + ((c ^ (r & 7)) << 3); }
template <typename T, typename SrcFn>
__device__ __forceinline__ void stage_rows64_raw(T* X16, int rows16, int n_rows, int lane, SrcFn src) {
    const int rsub = lane >> 3, c8 = lane & 7;
#pragma unroll 4
    for (int i = 0; i < kUW / 4; ++i) {
        const int r = 4 * i + rsub;
        if (r < rows16) {
            T* dst = X16 + swz64(r, c8);
            if (r < n_rows) cp_async16_cg(dst, src(r) + c8 * 8);
            else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
}
// ICT consecutive 16-bit elements, unconverted
template <typename T, int ICT> __device__ __forceinline__ void load_raw(const T* p, unsigned short (&w)[ICT]) {
    if constexpr (ICT == 4) {
        const uint2 v = *reinterpret_cast<const uint2*>(p);
        w[0] = (unsigned short)(v.x & 0xffffu);
        w[1] = (unsigned short)(v.x >> 16);
        w[2] = (unsigned short)(v.y & 0xffffu);
        w[3] = (unsigned short)(v.y >> 16);
    } else {
#pragma unroll
        for (int k = 0; k < ICT; ++k) w[k] = reinterpret_cast<const unsigned short*>(p)[k];
    }
}
__device__ __forceinline__ unsigned lds32(unsigned addr) {
    unsigned v;
    asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}

template <typename T, int ICT> __device__ __forceinline__ void load_w(const T* p, float (&w)[ICT]) {
    if constexpr (ICT == 4) {
        const float4 v = ld4(p);
        w[0] = v.x;
        w[1] = v.y;
        w[2] = v.z;
        w[3] = v.w;
    } else {
#pragma unroll
        for (int k = 0; k < ICT; ++k) w[k] = Elem<T>::up(p[k]);
    }
}
template <typename T, int ICT> __device__ __forceinline__ void store_w(T* p, const float (&w)[ICT]) {
    if constexpr (ICT == 4) {
        st4(p, make_float4(w[0], w[1], w[2], w[3]));
    } else {
#pragma unroll
        for (int k = 0; k < ICT; ++k) p[k] = Elem<T>::down(w[k]);
    }
}

// Merge rows that share next to nothing (random tables): staging their distinct feature rows 32 at a time
// costs more than it saves.  Every lane takes two channels of a 64-channel group and walks the 8 x m edges
// directly: feature rows from global memory (contiguous across the warp), indices from the landing area,
// weights as warp-wide broadcast loads.  Out of line, so that it does not weigh on the staged path's registers.
// more distinct feature rows than this in a tile (of at most 384): gather them unstaged.  Measured break-even:
// the staged path at about 170 distinct rows costs half of the unstaged one in fp32, less still for 16-bit
// inputs (whose staged products are cheap)
constexpr int kDirectUW = 288, kDirectUW16 = 352;
template <typename T, int ICT>
__device__ __noinline__ void wf_sum_unstaged(const long long* ring, const int* rowsS, const T* __restrict__ Wb,
                                             const T* __restrict__ Fb, T* __restrict__ Ob, int n, int m, int c,
                                             int lane) {
    for (int q = 0; q < kT; ++q) {
        const int rq = rowsS[q];
        if (rq < 0) continue;
        const T* wrow = Wb + (long long)rq * m * ICT;
        for (int c0 = 0; c0 < c; c0 += kCG) {
            const int ch = c0 + 2 * lane;
            float acc[ICT][2];
#pragma unroll
            for (int k = 0; k < ICT; ++k) acc[k][0] = acc[k][1] = 0.f;
#pragma unroll 4
            for (int j = 0; j < m; ++j) {
                const long long t = ring[q * m + j];
                if (t >= 0 && t < n) {
                    const T* fp = Fb + t * c + ch;
                    const float x0 = Elem<T>::up(fp[0]), x1 = Elem<T>::up(fp[1]);
                    float w[ICT];
                    load_w<T, ICT>(wrow + j * ICT, w);
#pragma unroll
                    for (int k = 0; k < ICT; ++k) {
                        acc[k][0] += w[k] * x0;
                        acc[k][1] += w[k] * x1;
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < ICT; ++k) {
                T* op = Ob + ((long long)rq * ICT + k) * c + ch;
                op[0] = Elem<T>::down(acc[k][0]);
                op[1] = Elem<T>::down(acc[k][1]);
            }
        }
    }
}

// MODE 0: wf_sum, MODE 1: wf_dot.  ICT = ic (1, 2 or 4).  c must be a multiple of 64.
// M48: m = 48 is known at compile time (every AutoFocusFormer merge table); C64: c = 64 (the first merge)
template <typename T, int MODE, int ICT, bool M48, bool C64>
__global__ void __launch_bounds__(32 * kWarps, 3)
wf_tiles_kernel(const WfParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    using WS = WfSmem<MODE>;
    constexpr bool kSplit = std::is_same<T, float>::value;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    unsigned char* base = smem_raw + size_t(warp) * WS::kTotal;
    float* Xs = reinterpret_cast<float*>(base);
    float* Op = reinterpret_cast<float*>(base + WS::kX);
    unsigned short* lut = reinterpret_cast<unsigned short*>(base + WS::kX + WS::kOp);
    unsigned short* uniq = lut + kE;
    int* rowsS = reinterpret_cast<int*>(uniq + kE);
    long long* ring = reinterpret_cast<long long*>(Xs);
    DedupScratch ds;
    ds.tok = reinterpret_cast<unsigned short*>(base + kE * 8);
    ds.uniq = uniq;
    ds.bm = reinterpret_cast<unsigned*>(Op);
    ds.pre = reinterpret_cast<unsigned short*>(ds.bm + kBMW);
    ds.rowbm = reinterpret_cast<unsigned*>(ds.pre + kBMW);

    const int m = M48 ? kMmax : p.m, c = C64 ? kCG : p.c, n = p.n, n_out = p.n_out;
    const int E = kT * m;
    const T* Fg = static_cast<const T*>(p.F);

    // fragment addresses (bytes in shared memory), fixed per lane
    unsigned xa[4][2];          // MODE 0: A = X^T, &Xs[t][16 mt + 8 h + g]
    unsigned wa = 0;            // MODE 0: B = Wd^T, &Wd[g][t]
    unsigned ya[2];             // MODE 1: A = gradient tile, &Ys[16 mt + g][t]
    unsigned xb[4][2];          // MODE 1: B = X^T, &Xs[g][8 ks + 4 h + t] for ks % 4 = 0..3
    if (MODE == 0) {
#pragma unroll
        for (int mt = 0; mt < 4; ++mt)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int col = 16 * mt + 8 * h + g;
                xa[mt][h] = smem_u32(Xs + t * kCG + ((((col >> 2) ^ (t << 1)) << 2) + (col & 3)));
            }
        wa = smem_u32(Op + g * kDL + t);
    } else {
        ya[0] = smem_u32(Op + g * kGL + t);
        ya[1] = smem_u32(Op + (16 + g) * kGL + t);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
#pragma unroll
            for (int h = 0; h < 2; ++h) xb[ks][h] = smem_u32(Xs + g * kCG + ((((2 * ks + h) ^ g) << 2) + t));
    }

    const unsigned total = (unsigned)p.batch * (unsigned)p.tiles;
    const unsigned nwarps = gridDim.x * kWarps;
    for (unsigned task = blockIdx.x * kWarps + warp; task < total; task += nwarps) {
        const int b = (int)(task / (unsigned)p.tiles);
        const int i0 = (int)(task - (unsigned)b * (unsigned)p.tiles) * kT;
        const long long brow = (long long)b * n_out;
        // ---- the tile's rows, their indices -> ring [8][m]
        __syncwarp();
        if (lane < kT) {
            int r = -1;
            if (i0 + lane < n_out) r = p.order ? p.order[brow + i0 + lane] : i0 + lane;
            if ((unsigned)r >= (unsigned)n_out) r = -1;     // an entry that is no row number: treated as absent
            rowsS[lane] = r;
        }
        __syncwarp();
#pragma unroll
        for (int q = 0; q < kT; ++q) {
            const int rq = rowsS[q];
            if (rq >= 0) {
                const int64_t* src = p.idx + (brow + rq) * m;
                for (int j = lane; j < m; j += 32) cp_async8_ca(ring + q * m + j, src + j);
                if (MODE == 0) {        // the row's weights will be wanted soon
                    const char* wrow = reinterpret_cast<const char*>(static_cast<const T*>(p.W) + (brow + rq) * m * ICT);
                    if (lane * 128 < m * ICT * (int)sizeof(T)) prefetch_l2(wrow + lane * 128);
                }
            } else {
                for (int j = lane; j < m; j += 32) ring[q * m + j] = -1;
            }
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncwarp();
        bool rowdup = false;
        const int U = dedup_tile(ds, ring, lut, E, m, 0, kT, MODE == 0, &rowdup, lane, n);
        if (MODE == 0 && U > (kSplit ? kDirectUW : kDirectUW16)) {
            wf_sum_unstaged<T, ICT>(ring, rowsS, static_cast<const T*>(p.W) + brow * m * ICT, Fg + (long long)b * n * c,
                                    static_cast<T*>(p.out) + brow * ICT * c, n, m, c, lane);
            continue;
        }
        // ---- per edge of this lane: offset of its weights; tile row into lut
        int woff[kEPL];
        {
            int q = 0, j = lane;
            while (j >= m) { j -= m; ++q; }
#pragma unroll
            for (int i = 0; i < kEPL; ++i) {
                const int x = lane + 32 * i;
                woff[i] = -1;
                if (x < E) {
                    const int rq = rowsS[q];
                    if (rq >= 0) woff[i] = (rq * m + j) * ICT;
                    const unsigned short s = lut[x];
                    if (s != kSkip) lut[x] = (unsigned short)(s | (q << 12));
                    j += 32;
                    while (j >= m) { j -= m; ++q; }
                }
            }
        }
        __syncwarp();
        const int nchunks = (U + kUW - 1) / kUW;

        if (MODE == 0) {
            const T* Wb = static_cast<const T*>(p.W) + brow * m * ICT;
            T* Ob = static_cast<T*>(p.out) + brow * ICT * c;
            float* Wd = Op;
            for (int c0 = 0; c0 < c; c0 += kCG) {
                const T* Fb = Fg + (long long)b * n * c + c0;
                float acc[ICT][4][4];
#pragma unroll
                for (int k = 0; k < ICT; ++k)
#pragma unroll
                    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
                        for (int i = 0; i < 4; ++i) acc[k][mt][i] = 0.f;
                for (int ch = 0; ch < nchunks; ++ch) {
                    const int u0 = ch * kUW;
                    const int Uc = min(kUW, U - u0);
                    const int rows8 = (Uc + 7) & ~7;
                    __syncwarp();
                    if (!kSplit && !rowdup) {
                        // 16-bit inputs stay 16-bit: m16n8k16 products, A = X^T through ldmatrix.trans
                        const int rows16 = (Uc + 15) & ~15;
                        T* X16 = reinterpret_cast<T*>(Xs);
                        unsigned short* Wd16 = reinterpret_cast<unsigned short*>(Op);
                        stage_rows64_raw<T>(X16, rows16, Uc, lane,
                                            [&](int r) { return Fb + (long long)uniq[u0 + r] * c; });
                        cp_async_commit();
                        for (int z = lane; z < ICT * kT * kDL16 * 2 / 16; z += 32)
                            reinterpret_cast<float4*>(Wd16)[z] = make_float4(0.f, 0.f, 0.f, 0.f);
                        __syncwarp();
#pragma unroll
                        for (int i = 0; i < kEPL; ++i) {
                            const int x = lane + 32 * i;
                            if (x < E) {
                                const unsigned short lr = lut[x];
                                const int rel = (int)(lr & 0xfffu) - u0;
                                if (lr != kSkip && rel >= 0 && rel < Uc && woff[i] >= 0) {
                                    unsigned short w[ICT];
                                    load_raw<T, ICT>(Wb + woff[i], w);
#pragma unroll
                                    for (int k = 0; k < ICT; ++k) Wd16[(k * kT + (lr >> 12)) * kDL16 + rel] = w[k];
                                }
                            }
                        }
                        cp_async_wait<0>();
                        __syncwarp();
                        const int mi = lane >> 3, rr = lane & 7;
                        unsigned xa16[4];
#pragma unroll
                        for (int mt = 0; mt < 4; ++mt) xa16[mt] = smem_u32(X16 + swz64((mi >> 1) * 8 + rr, 2 * mt + (mi & 1)));
                        const unsigned wa16 = smem_u32(Wd16 + g * kDL16 + 2 * t);
                        for (int ks = 0; ks < (rows16 >> 4); ++ks) {
                            unsigned a[4][4];
#pragma unroll
                            for (int mt = 0; mt < 4; ++mt) ldsm_x4_trans(a[mt], xa16[mt] + ks * 16 * kCG * 2);
#pragma unroll
                            for (int k = 0; k < ICT; ++k) {
                                unsigned bq[2];
                                bq[0] = lds32(wa16 + (k * kT * kDL16 + 16 * ks) * 2);
                                bq[1] = lds32(wa16 + (k * kT * kDL16 + 16 * ks + 8) * 2);
#pragma unroll
                                for (int mt = 0; mt < 4; ++mt) mma16(acc[k][mt], a[mt], bq, static_cast<const T*>(nullptr));
                            }
                        }
                        continue;
                    }
                    stage_rows64<T, 0>(Xs, rows8, Uc, lane,
                                       [&](int r) { return Fb + (long long)uniq[u0 + r] * c; });
                    cp_async_commit();
                    for (int z = lane; z < ICT * kT * kDL / 4; z += 32)
                        reinterpret_cast<float4*>(Wd)[z] = make_float4(0.f, 0.f, 0.f, 0.f);
                    __syncwarp();
                    if (!rowdup) {
#pragma unroll
                        for (int i0e = 0; i0e < kEPL; i0e += 4) {
                            float w[4][ICT];
                            int dst[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int x = lane + 32 * (i0e + i);
                                dst[i] = -1;
                                if (x < E) {
                                    const unsigned short lr = lut[x];
                                    const int rel = (int)(lr & 0xfffu) - u0;
                                    if (lr != kSkip && rel >= 0 && rel < Uc && woff[i0e + i] >= 0) {
                                        dst[i] = (lr >> 12) * kDL + rel;
                                        load_w<T, ICT>(Wb + woff[i0e + i], w[i]);
                                    }
                                }
                            }
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                if (dst[i] >= 0) {
#pragma unroll
                                    for (int k = 0; k < ICT; ++k) Wd[k * kT * kDL + dst[i]] = w[i][k];
                                }
                        }
                    } else if (lane < kT && rowsS[lane] >= 0) {
                        // some row repeats a neighbour: one lane per row adds its weights in column order
                        const T* wrow = Wb + (long long)rowsS[lane] * m * ICT;
#pragma unroll 1
                        for (int j = 0; j < m; ++j) {
                            const unsigned short lr = lut[lane * m + j];
                            const int rel = (int)(lr & 0xfffu) - u0;
                            if (lr != kSkip && rel >= 0 && rel < Uc) {
#pragma unroll
                                for (int k = 0; k < ICT; ++k)
                                    Wd[(k * kT + lane) * kDL + rel] += Elem<T>::up(wrow[j * ICT + k]);
                            }
                        }
                    }
                    cp_async_wait<0>();
                    __syncwarp();
                    // D_k[ch][q] += sum_u X[u][ch] * Wd[k 8 + q][u]
                    for (int us = 0; us < rows8; us += 8) {
                        unsigned ah[4][4], al[4][4];
#pragma unroll
                        for (int mt = 0; mt < 4; ++mt) {
                            float a[4];
                            const unsigned a0 = xa[mt][0] + us * (kCG * 4), a1 = xa[mt][1] + us * (kCG * 4);
                            WF_LDS(a[0], a0, 0);
                            WF_LDS(a[1], a1, 0);
                            WF_LDS(a[2], a0, 4 * kCG * 4);
                            WF_LDS(a[3], a1, 4 * kCG * 4);
#pragma unroll
                            for (int i = 0; i < 4; ++i) wf_split<kSplit>(a[i], ah[mt][i], al[mt][i]);
                        }
                        const unsigned w0 = wa + us * 4;
#pragma unroll
                        for (int k = 0; k < ICT; ++k) {
                            float bv[2];
                            WF_LDS(bv[0], w0, k * kT * kDL * 4);
                            WF_LDS(bv[1], w0, k * kT * kDL * 4 + 16);
                            unsigned bh[2], bl[2];
                            wf_split<kSplit>(bv[0], bh[0], bl[0]);
                            wf_split<kSplit>(bv[1], bh[1], bl[1]);
                            wf_mma_row<kSplit, 4>(acc[k], ah, al, bh, bl);
                        }
                    }
                }
                // D fragments -> output tile [8][kGL] in X -> 16-byte stores, one ic at a time
                float* Ot = Xs;
#pragma unroll
                for (int k = 0; k < ICT; ++k) {
                    __syncwarp();
#pragma unroll
                    for (int mt = 0; mt < 4; ++mt) {
                        float* o = Ot + (2 * t) * kGL + 16 * mt + g;
                        o[0] = acc[k][mt][0];
                        o[kGL] = acc[k][mt][1];
                        o[8] = acc[k][mt][2];
                        o[kGL + 8] = acc[k][mt][3];
                    }
                    __syncwarp();
                    const int rsub = lane >> 4, chn = lane & 15;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int q = 2 * i + rsub;
                        const int rq = rowsS[q];
                        if (rq >= 0)
                            st4(Ob + ((long long)rq * ICT + k) * c + c0 + chn * 4,
                                *reinterpret_cast<const float4*>(Ot + q * kGL + chn * 4));
                    }
                }
            }
        } else {
            T* Wout = static_cast<T*>(p.out) + brow * m * ICT;
            const T* Gb = static_cast<const T*>(p.G) + brow * ICT * c;
            float* Ys = Op;
            float* Sb = Xs;
            // edges without a neighbour get zero
            {
                float z[ICT];
#pragma unroll
                for (int k = 0; k < ICT; ++k) z[k] = 0.f;
#pragma unroll
                for (int i = 0; i < kEPL; ++i) {
                    const int x = lane + 32 * i;
                    if (x < E && woff[i] >= 0 && lut[x] == kSkip) store_w<T, ICT>(Wout + woff[i], z);
                }
            }
            const bool multi = c > kCG;          // several channel groups: the gradient tile is staged per group
            for (int ch = 0; ch < nchunks; ++ch) {
                const int u0 = ch * kUW;
                const int Uc = min(kUW, U - u0);
                const int rows8 = (Uc + 7) & ~7;
                constexpr int MT = (ICT * kT + 15) / 16;
                float acc[MT][4][4];
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                        for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.f;
                for (int c0 = 0; c0 < c; c0 += kCG) {
                    const T* Fb = Fg + (long long)b * n * c + c0;
                    __syncwarp();
                    if constexpr (!kSplit) {
                        // 16-bit inputs stay 16-bit: A = gradient tile and B = X^T, both through ldmatrix
                        const int rows16 = (Uc + 15) & ~15;
                        T* X16 = reinterpret_cast<T*>(Xs);
                        T* Y16 = reinterpret_cast<T*>(Op);
                        stage_rows64_raw<T>(X16, rows16, Uc, lane,
                                            [&](int r) { return Fb + (long long)uniq[u0 + r] * c; });
                        if (ch == 0 || multi) {
                            const int rsub = lane >> 3, c8 = lane & 7;
#pragma unroll 2
                            for (int i = 0; i < MT * 16 / 4; ++i) {
                                const int r = 4 * i + rsub;                       // k 8 + q
                                const int rq = r < ICT * kT ? rowsS[r & 7] : -1;
                                T* dst = Y16 + swz64(r, c8);
                                if (rq >= 0) cp_async16_cg(dst, Gb + ((long long)rq * ICT + (r >> 3)) * c + c0 + c8 * 8);
                                else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
                            }
                        }
                        cp_async_commit();
                        cp_async_wait<0>();
                        __syncwarp();
                        const int mi = lane >> 3, rr = lane & 7;
                        unsigned afr[MT][4][4];
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                            for (int ks = 0; ks < 4; ++ks)
                                ldsm_x4(afr[mt][ks], smem_u32(Y16 + swz64(16 * mt + (mi & 1) * 8 + rr, 2 * ks + (mi >> 1))));
#pragma unroll
                        for (int nt = 0; nt < 4; ++nt) {
                            if (nt * 8 < rows16) {
                                unsigned bfr[2][4];
#pragma unroll
                                for (int h = 0; h < 2; ++h) ldsm_x4(bfr[h], smem_u32(X16 + swz64(8 * nt + rr, 4 * h + mi)));
#pragma unroll
                                for (int ks = 0; ks < 4; ++ks) {
                                    const unsigned bq[2] = {bfr[ks >> 1][(ks & 1) * 2], bfr[ks >> 1][(ks & 1) * 2 + 1]};
#pragma unroll
                                    for (int mt = 0; mt < MT; ++mt)
                                        mma16(acc[mt][nt], afr[mt][ks], bq, static_cast<const T*>(nullptr));
                                }
                            }
                        }
                        continue;
                    }
                    stage_rows64<T, 1>(Xs, rows8, Uc, lane,
                                       [&](int r) { return Fb + (long long)uniq[u0 + r] * c; });
                    if (ch == 0 || multi) {
                        // gradient tile: row k 8 + q <- d_feat_new[b, row q, k, c0 .. c0 + 63]
                        if constexpr (std::is_same<T, float>::value) {
                            const int rsub = lane >> 4, chn = lane & 15;
#pragma unroll 4
                            for (int i = 0; i < ICT * kT / 2; ++i) {
                                const int r = 2 * i + rsub;              // k 8 + q
                                const int rq = rowsS[r & 7];
                                float* dst = Ys + r * kGL + chn * 4;
                                if (rq >= 0) cp_async16_cg(dst, Gb + ((long long)rq * ICT + (r >> 3)) * c + c0 + chn * 4);
                                else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
                            }
                        } else {
                            const int rsub = lane >> 3, c8 = lane & 7;
#pragma unroll 2
                            for (int i = 0; i < ICT * kT / 4; ++i) {
                                const int r = 4 * i + rsub;
                                const int rq = rowsS[r & 7];
                                float4 va = make_float4(0.f, 0.f, 0.f, 0.f), vb = va;
                                if (rq >= 0)
                                    up8(*reinterpret_cast<const uint4*>(Gb + ((long long)rq * ICT + (r >> 3)) * c + c0 + c8 * 8),
                                        static_cast<const T*>(nullptr), va, vb);
                                *reinterpret_cast<float4*>(Ys + r * kGL + c8 * 8) = va;
                                *reinterpret_cast<float4*>(Ys + r * kGL + c8 * 8 + 4) = vb;
                            }
                        }
                    }
                    cp_async_commit();
                    cp_async_wait<0>();
                    __syncwarp();
                    // S[k 8 + q][u] += sum_ch Ys[k 8 + q][ch] * X[u][ch]
#pragma unroll
                    for (int ks = 0; ks < kCG / 8; ++ks) {
                        unsigned ah[MT][4], al[MT][4];
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            float a[4];
                            WF_LDS(a[0], ya[mt], ks * 32);
                            WF_LDS(a[1], ya[mt], ks * 32 + 8 * kGL * 4);
                            WF_LDS(a[2], ya[mt], ks * 32 + 16);
                            WF_LDS(a[3], ya[mt], ks * 32 + 8 * kGL * 4 + 16);
#pragma unroll
                            for (int i = 0; i < 4; ++i) wf_split<kSplit>(a[i], ah[mt][i], al[mt][i]);
                        }
#pragma unroll
                        for (int nt = 0; nt < 4; ++nt) {
                            if (nt * 8 < rows8) {
                                float bv[2];
                                WF_LDS(bv[0], xb[ks & 3][0], nt * 8 * kCG * 4 + (ks >> 2) * 128);
                                WF_LDS(bv[1], xb[ks & 3][1], nt * 8 * kCG * 4 + (ks >> 2) * 128);
                                unsigned bh[2], bl[2];
                                wf_split<kSplit>(bv[0], bh[0], bl[0]);
                                wf_split<kSplit>(bv[1], bh[1], bl[1]);
                                if (kSplit) {
#pragma unroll
                                    for (int mt = 0; mt < MT; ++mt) mma_tf32(acc[mt][nt], al[mt], bh);
#pragma unroll
                                    for (int mt = 0; mt < MT; ++mt) mma_tf32(acc[mt][nt], ah[mt], bl);
                                }
#pragma unroll
                                for (int mt = 0; mt < MT; ++mt) mma_tf32(acc[mt][nt], ah[mt], bh);
                            }
                        }
                    }
                }
                __syncwarp();                               // every lane is done with X: the scores go there
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt) {
                        float* sp = Sb + (16 * mt + g) * kDL + 8 * nt + 2 * t;
                        *reinterpret_cast<float2*>(sp) = make_float2(acc[mt][nt][0], acc[mt][nt][1]);
                        *reinterpret_cast<float2*>(sp + 8 * kDL) = make_float2(acc[mt][nt][2], acc[mt][nt][3]);
                    }
                __syncwarp();
                // every edge whose neighbour is in this stage picks its ic scores
#pragma unroll
                for (int i = 0; i < kEPL; ++i) {
                    const int x = lane + 32 * i;
                    if (x < E && woff[i] >= 0) {
                        const unsigned short lr = lut[x];
                        const int rel = (int)(lr & 0xfffu) - u0;
                        if (lr != kSkip && rel >= 0 && rel < Uc) {
                            float w[ICT];
#pragma unroll
                            for (int k = 0; k < ICT; ++k) w[k] = Sb[(k * kT + (lr >> 12)) * kDL + rel];
                            store_w<T, ICT>(Wout + woff[i], w);
                        }
                    }
                }
            }
        }
    }
}

// ----------------------------------------------------------------------------- d_feat
//   d_feat[b, t, :] = sum over inverse-index entries (i, j) of target t and k < ic:
//                     w[b, i, j, k] * d_feat_new[b, i, k, :]
// A warp takes 8 consecutive targets, concatenates their segments (256 entries at a time) and
// de-duplicates the merge ROWS i.  The ic gradient rows of a merge row are contiguous in memory and so
// are the ic weights of an entry: the rows are staged as [32 / ic merge rows x ic][64 channels], the
// weights go into the dense [8 targets x 32] tile with one 16-byte copy per entry (ic = 4), and the
// product needs a single 8-wide N tile, so the accumulators are 16 registers.  The reference adds
// every (entry, ic, channel) term with atomicAdd (clusten/src/clustenwf_cuda_kernel.cu:121-131).
struct WfScatterParams {
    const void* W;        // weights [b, n_out, m, ic]
    const void* G;        // d_feat_new [b, n_out, ic, c]
    void* out;            // d_feat [b, n, c]
    const int64_t* idx;   // [b, n_out, m]
    InverseView inv;
    int batch, n_out, n, m, c, tiles;
    unsigned m_magic, m_shift;            // x / m = (umulhi(magic, x) + x) >> shift
};
constexpr int kEE = 192;                  // entries handled at a time (sized so that five CTAs fit on an SM)
constexpr int kUD = 32;                   // gradient rows per stage (24 rows and six CTAs per SM measured slower)
struct WfScatterSmem {
    static constexpr int kX = kUD * kCG * 4;
    static constexpr int kOp = kT * kWLD * 4;     // dense weights [8][kDL]; bitmap scratch before that
    static constexpr int kEnt = kEE * 4;          // row * m + slot of each entry (bit 31: the row repeats the target)
    static constexpr int kLut = kEE * 2;          // entry -> slot | tile row << 12;  slot -> merge row
    static constexpr int kTotal = kX + kOp + kEnt + 2 * kLut;
};
static_assert(kBMW * 4 + kBMW * 2 + (kE / 32) * 4 <= kT * kWLD * 4 && kT * kDL <= kT * kWLD, "scratch must fit in Op");
static_assert(kEE * 4 <= kUD * kCG * 4 && kT * kGL * 4 <= kUD * kCG * 4 && ((kUD + 15) & ~15) * kCG * 2 <= kUD * kCG * 4,
              "token scratch, output tile and padded 16-bit rows must fit in the row buffer");

template <typename T, int ICT, bool M48, bool C64>
__global__ void __launch_bounds__(32 * kWarps, 5)
wf_dfeat_kernel(const WfScatterParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    using WS = WfScatterSmem;
    constexpr bool kSplit = std::is_same<T, float>::value;
    constexpr int kRowsPer = kUD / ICT;          // merge rows per stage
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    unsigned char* base = smem_raw + size_t(warp) * WS::kTotal;
    float* Xs = reinterpret_cast<float*>(base);
    float* Wd = reinterpret_cast<float*>(base + WS::kX);
    unsigned* ent = reinterpret_cast<unsigned*>(base + WS::kX + WS::kOp);
    unsigned short* lut = reinterpret_cast<unsigned short*>(base + WS::kX + WS::kOp + WS::kEnt);
    unsigned short* uniq = lut + kEE;
    DedupScratch ds;
    ds.tok = reinterpret_cast<unsigned short*>(base);
    ds.uniq = uniq;
    ds.bm = reinterpret_cast<unsigned*>(Wd);
    ds.pre = reinterpret_cast<unsigned short*>(ds.bm + kBMW);
    ds.rowbm = reinterpret_cast<unsigned*>(ds.pre + kBMW);
    const int m = M48 ? kMmax : p.m, c = C64 ? kCG : p.c, n_out = p.n_out, n_tgt = p.n;
    auto div_m = [&](unsigned x) { return M48 ? x / 48u : fast_div_u(x, p.m_magic, p.m_shift); };
    const T* Wg = static_cast<const T*>(p.W);
    const T* Gg = static_cast<const T*>(p.G);
    T* Og = static_cast<T*>(p.out);

    unsigned xa[4][2];
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int col = 16 * mt + 8 * h + g;
            xa[mt][h] = smem_u32(Xs + t * kCG + ((((col >> 2) ^ (t << 1)) << 2) + (col & 3)));
        }
    const unsigned wa = smem_u32(Wd + g * kDL + t);

    const unsigned total = (unsigned)p.batch * (unsigned)p.tiles;
    const unsigned nwarps = gridDim.x * kWarps;
    auto load_segment = [&](unsigned task, int& len, int& start) {
        len = 0;
        start = 0;
        if (task < total) {
            const int b = (int)(task / (unsigned)p.tiles);
            const int tt = (int)(task - (unsigned)b * (unsigned)p.tiles) * kT + lane;
            if (lane < kT && tt < n_tgt) {
                len = p.inv.seglen[(long long)b * n_tgt + tt];
                start = p.inv.rowptr[(long long)b * (n_tgt + 1) + tt];
            }
        }
    };
    int next_len, next_start;
    load_segment(blockIdx.x * kWarps + warp, next_len, next_start);
    for (unsigned task = blockIdx.x * kWarps + warp; task < total; task += nwarps) {
        const int b = (int)(task / (unsigned)p.tiles);
        const int t0 = (int)(task - (unsigned)b * (unsigned)p.tiles) * kT;
        const long long brow = (long long)b * n_out;
        const int64_t* idx_b = p.idx + brow * m;
        const int* entries = p.inv.entries + brow * m;
        const T* Wb = Wg + brow * m * ICT;
        const T* Gb = Gg + brow * ICT * c;
        T* Ob = Og + (long long)b * n_tgt * c;
        const int len = next_len, start = next_start;
        load_segment(task + nwarps, next_len, next_start);
        int incl = len;
#pragma unroll
        for (int o = 1; o < kT; o <<= 1) {
            const int y = __shfl_up_sync(kFull, incl, o);
            if (lane >= o) incl += y;
        }
        const int E_total = __shfl_sync(kFull, incl, kT - 1);
        int off[kT], st[kT];
#pragma unroll
        for (int r = 0; r < kT; ++r) {
            off[r] = __shfl_sync(kFull, incl - len, r);
            st[r] = __shfl_sync(kFull, start, r);
        }
        unsigned pk[kT];                                        // (segment start - offset) << 3 | tile row
#pragma unroll
        for (int r = 0; r < kT; ++r) pk[r] = ((unsigned)(st[r] - off[r]) << 3) | (unsigned)r;
        for (int e0 = 0; e0 == 0 || e0 < E_total; e0 += kEE) {
            const int E = max(0, min(kEE, E_total - e0));
            int lo = INT_MAX, hi = -1;
            bool any_flag = false;
            __syncwarp();
#pragma unroll 4
            for (int x = lane; x < E; x += 32) {
                const int pe = e0 + x;
                // (segment start - offset in the edge list) and the tile row travel through one select chain
                unsigned v = pk[0];
#pragma unroll
                for (int j = 1; j < kT; ++j) v = pe >= off[j] ? pk[j] : v;
                const int r = (int)(v & 7u);
                const unsigned e = (unsigned)__ldg(entries + (int)(v >> 3) + pe);
                const int row = (int)div_m(e & ~kDupFlag);
                ent[x] = e;
                ds.tok[x] = (unsigned short)row;
                lut[x] = (unsigned short)(r << 12);
                lo = min(lo, row);
                hi = max(hi, row);
                any_flag = any_flag || (e & kDupFlag) != 0u;
            }
            any_flag = __any_sync(kFull, any_flag);
            int U = 0;
            if (E > 0) {
                bool unused = false;
                unsigned short* slots = ds.tok + kEE;
                U = dedup_tokens(ds, slots, E, m, false, &unused, lane, lo, hi);
                for (int x = lane; x < E; x += 32) lut[x] = (unsigned short)(lut[x] | slots[x]);
            }
            __syncwarp();
            for (int c0 = 0; c0 < c; c0 += kCG) {
                float acc[4][4];
#pragma unroll
                for (int mt = 0; mt < 4; ++mt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[mt][i] = 0.f;
                for (int u0 = 0; u0 < U; u0 += kRowsPer) {
                    const int Uc = min(kRowsPer, U - u0);           // merge rows of this stage
                    const int nrows = Uc * ICT;
                    const int rows8 = (nrows + 7) & ~7;
                    __syncwarp();
                    if (!kSplit && !any_flag) {
                        // 16-bit inputs stay 16-bit (no weight of this chunk is a sum over repeated slots)
                        const int rows16 = (nrows + 15) & ~15;
                        T* X16 = reinterpret_cast<T*>(Xs);
                        unsigned short* Wd16 = reinterpret_cast<unsigned short*>(Wd);
                        stage_rows64_raw<T>(X16, rows16, nrows, lane, [&](int r) {
                            return Gb + ((long long)uniq[u0 + r / ICT] * ICT + (r % ICT)) * c + c0;
                        });
                        cp_async_commit();
                        for (int z = lane; z < kT * kDL16 * 2 / 16; z += 32)
                            reinterpret_cast<float4*>(Wd16)[z] = make_float4(0.f, 0.f, 0.f, 0.f);
                        __syncwarp();
#pragma unroll 4
                        for (int x = lane; x < E; x += 32) {
                            const unsigned lr = lut[x];
                            const int rel = (int)(lr & 0xfffu) - u0;
                            if (rel >= 0 && rel < Uc) {
                                unsigned short w[ICT];
                                load_raw<T, ICT>(Wb + (size_t)ent[x] * ICT, w);
#pragma unroll
                                for (int k = 0; k < ICT; ++k) Wd16[(lr >> 12) * kDL16 + rel * ICT + k] = w[k];
                            }
                        }
                        cp_async_wait<0>();
                        __syncwarp();
                        const int mi = lane >> 3, rr = lane & 7;
                        const unsigned wa16 = smem_u32(Wd16 + g * kDL16 + 2 * t);
                        for (int ks = 0; ks < (rows16 >> 4); ++ks) {
                            unsigned bq[2];
                            bq[0] = lds32(wa16 + 16 * ks * 2);
                            bq[1] = lds32(wa16 + (16 * ks + 8) * 2);
#pragma unroll
                            for (int mt = 0; mt < 4; ++mt) {
                                unsigned a[4];
                                ldsm_x4_trans(a, smem_u32(X16 + swz64((mi >> 1) * 8 + rr, 2 * mt + (mi & 1))) + ks * 16 * kCG * 2);
                                mma16(acc[mt], a, bq, static_cast<const T*>(nullptr));
                            }
                        }
                        continue;
                    }
                    for (int z = lane; z < kT * kDL / 4; z += 32)
                        reinterpret_cast<float4*>(Wd)[z] = make_float4(0.f, 0.f, 0.f, 0.f);
                    __syncwarp();
                    // the ic weights of every entry whose merge row is in this stage
#pragma unroll 4
                    for (int x = lane; x < E; x += 32) {
                        const unsigned lr = lut[x];
                        const int rel = (int)(lr & 0xfffu) - u0;
                        if (rel >= 0 && rel < Uc) {
                            const unsigned e = ent[x];
                            float* dst = Wd + (lr >> 12) * kDL + rel * ICT;
                            if (!(e & kDupFlag)) {
                                if (kSplit && ICT == 4) {
                                    cp_async16_ca(dst, Wb + (size_t)e * ICT);
                                } else {
                                    float w[ICT];
                                    load_w<T, ICT>(Wb + (size_t)e * ICT, w);
#pragma unroll
                                    for (int k = 0; k < ICT; ++k) dst[k] = w[k];
                                }
                            } else {
                                // the merge row names the target several times: add its slots in order
                                const unsigned row = div_m(e & ~kDupFlag);
                                const int64_t* irow = idx_b + (long long)row * m;
                                float w[ICT];
#pragma unroll
                                for (int k = 0; k < ICT; ++k) w[k] = 0.f;
#pragma unroll 1
                                for (int j = 0; j < m; ++j)
                                    if (irow[j] == t0 + (int)(lr >> 12)) {
#pragma unroll
                                        for (int k = 0; k < ICT; ++k)
                                            w[k] += Elem<T>::up(Wb[((size_t)row * m + j) * ICT + k]);
                                    }
#pragma unroll
                                for (int k = 0; k < ICT; ++k) dst[k] = w[k];
                            }
                        }
                    }
                    stage_rows64<T, 0>(Xs, rows8, nrows, lane, [&](int r) {
                        return Gb + ((long long)uniq[u0 + r / ICT] * ICT + (r % ICT)) * c + c0;
                    });
                    cp_async_commit();
                    cp_async_wait<0>();
                    __syncwarp();
                    for (int us = 0; us < rows8; us += 8) {
                        float bv[2];
                        const unsigned w0 = wa + us * 4;
                        WF_LDS(bv[0], w0, 0);
                        WF_LDS(bv[1], w0, 16);
                        unsigned bh[2], bl[2];
                        wf_split<kSplit>(bv[0], bh[0], bl[0]);
                        wf_split<kSplit>(bv[1], bh[1], bl[1]);
                        unsigned ah[4][4], al[4][4];
#pragma unroll
                        for (int mt = 0; mt < 4; ++mt) {
                            float a[4];
                            const unsigned a0 = xa[mt][0] + us * (kCG * 4), a1 = xa[mt][1] + us * (kCG * 4);
                            WF_LDS(a[0], a0, 0);
                            WF_LDS(a[1], a1, 0);
                            WF_LDS(a[2], a0, 4 * kCG * 4);
                            WF_LDS(a[3], a1, 4 * kCG * 4);
#pragma unroll
                            for (int i = 0; i < 4; ++i) wf_split<kSplit>(a[i], ah[mt][i], al[mt][i]);
                        }
                        wf_mma_row<kSplit, 4>(acc, ah, al, bh, bl);
                    }
                }
                // D fragments -> output tile [8][kGL] in X -> 16-byte stores (added to what earlier chunks
                // of a long entry list wrote)
                float* Ot = Xs;
                __syncwarp();
#pragma unroll
                for (int mt = 0; mt < 4; ++mt) {
                    float* o = Ot + (2 * t) * kGL + 16 * mt + g;
                    o[0] = acc[mt][0];
                    o[kGL] = acc[mt][1];
                    o[8] = acc[mt][2];
                    o[kGL + 8] = acc[mt][3];
                }
                __syncwarp();
                const int rsub = lane >> 4, chn = lane & 15;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int q = 2 * i + rsub;
                    if (t0 + q < n_tgt) {
                        T* dstp = Ob + (long long)(t0 + q) * c + c0 + chn * 4;
                        float4 v = *reinterpret_cast<const float4*>(Ot + q * kGL + chn * 4);
                        if (e0 > 0) {
                            const float4 old = ld4(dstp);
                            v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
                        }
                        st4(dstp, v);
                    }
                }
                __syncwarp();
            }
        }
    }
}

// The same reduction without staging the gradient rows: a warp still takes 8 consecutive targets, lists their
// entries and de-duplicates the merge rows (about 18 per tile on AutoFocusFormer's tables), but then every lane
// owns 2 of the 64 channels for ALL 8 targets: per distinct merge row it reads its share of the ic gradient rows
// once (ic loads of 256 contiguous bytes per warp) and adds it into the 8 targets' accumulators with the row's
// weights, which sit in a dense [8 targets][32 rows][ic] fp32 tile in shared memory and are read as broadcasts.
// Plain FMAs in merge-row order: no tensor cores (nothing to split into TF32 passes), 5.5 KB of shared memory per
// warp instead of 11.4, 32 warps per SM instead of 20.
constexpr int kUR = 32;                   // distinct merge rows per pass of the dense weight tile
struct WfRowsSmem {
    static constexpr int kWd = kT * kUR * 4 * 4;  // dense weights [8][kUR][ic <= 4]; de-duplication scratch before that
    static constexpr int kEnt = kEE * 4;
    static constexpr int kLut = kEE * 2;
    static constexpr int kTotal = kWd + kEnt + 2 * kLut;
};
static_assert(kEE * 4 + kBMW * 4 + kBMW * 2 + (kE / 32) * 4 <= WfRowsSmem::kWd, "scratch must fit in the weight tile");

template <typename T, int ICT, bool M48, bool C64>
__global__ void __launch_bounds__(32 * kWarps, 8)
wf_dfeat_rows_kernel(const WfScatterParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    using WS = WfRowsSmem;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned char* base = smem_raw + size_t(warp) * WS::kTotal;
    float* Wd = reinterpret_cast<float*>(base);
    unsigned* ent = reinterpret_cast<unsigned*>(base + WS::kWd);
    unsigned short* lut = reinterpret_cast<unsigned short*>(base + WS::kWd + WS::kEnt);
    unsigned short* uniq = lut + kEE;
    DedupScratch ds;
    ds.tok = reinterpret_cast<unsigned short*>(base);
    ds.uniq = uniq;
    ds.bm = reinterpret_cast<unsigned*>(base + kEE * 4);
    ds.pre = reinterpret_cast<unsigned short*>(ds.bm + kBMW);
    ds.rowbm = reinterpret_cast<unsigned*>(ds.pre + kBMW);
    const int m = M48 ? kMmax : p.m, c = C64 ? kCG : p.c, n_out = p.n_out, n_tgt = p.n;
    auto div_m = [&](unsigned x) { return M48 ? x / 48u : fast_div_u(x, p.m_magic, p.m_shift); };
    const T* Wg = static_cast<const T*>(p.W);
    const T* Gg = static_cast<const T*>(p.G);
    T* Og = static_cast<T*>(p.out);

    const unsigned total = (unsigned)p.batch * (unsigned)p.tiles;
    const unsigned nwarps = gridDim.x * kWarps;
    auto load_segment = [&](unsigned task, int& len, int& start) {
        len = 0;
        start = 0;
        if (task < total) {
            const int b = (int)(task / (unsigned)p.tiles);
            const int tt = (int)(task - (unsigned)b * (unsigned)p.tiles) * kT + lane;
            if (lane < kT && tt < n_tgt) {
                len = p.inv.seglen[(long long)b * n_tgt + tt];
                start = p.inv.rowptr[(long long)b * (n_tgt + 1) + tt];
            }
        }
    };
    int next_len, next_start;
    load_segment(blockIdx.x * kWarps + warp, next_len, next_start);
    for (unsigned task = blockIdx.x * kWarps + warp; task < total; task += nwarps) {
        const int b = (int)(task / (unsigned)p.tiles);
        const int t0 = (int)(task - (unsigned)b * (unsigned)p.tiles) * kT;
        const long long brow = (long long)b * n_out;
        const int64_t* idx_b = p.idx + brow * m;
        const int* entries = p.inv.entries + brow * m;
        const T* Wb = Wg + brow * m * ICT;
        const T* Gb = Gg + brow * ICT * c + 2 * lane;
        T* Ob = Og + (long long)b * n_tgt * c + 2 * lane;
        const int len = next_len, start = next_start;
        load_segment(task + nwarps, next_len, next_start);
        int incl = len;
#pragma unroll
        for (int o = 1; o < kT; o <<= 1) {
            const int y = __shfl_up_sync(kFull, incl, o);
            if (lane >= o) incl += y;
        }
        const int E_total = __shfl_sync(kFull, incl, kT - 1);
        int off[kT], st[kT];
#pragma unroll
        for (int r = 0; r < kT; ++r) {
            off[r] = __shfl_sync(kFull, incl - len, r);
            st[r] = __shfl_sync(kFull, start, r);
        }
        unsigned pk[kT];                                        // (segment start - offset) << 3 | tile row
#pragma unroll
        for (int r = 0; r < kT; ++r) pk[r] = ((unsigned)(st[r] - off[r]) << 3) | (unsigned)r;
        for (int e0 = 0; e0 == 0 || e0 < E_total; e0 += kEE) {
            const int E = max(0, min(kEE, E_total - e0));
            int lo = INT_MAX, hi = -1;
            __syncwarp();
#pragma unroll 4
            for (int x = lane; x < E; x += 32) {
                const int pe = e0 + x;
                unsigned v = pk[0];
#pragma unroll
                for (int j = 1; j < kT; ++j) v = pe >= off[j] ? pk[j] : v;
                const int r = (int)(v & 7u);
                const unsigned e = (unsigned)__ldg(entries + (int)(v >> 3) + pe);
                const int row = (int)div_m(e & ~kDupFlag);
                ent[x] = e;
                ds.tok[x] = (unsigned short)row;
                lut[x] = (unsigned short)(r << 12);
                lo = min(lo, row);
                hi = max(hi, row);
            }
            int U = 0;
            if (E > 0) {
                bool unused = false;
                unsigned short* slots = ds.tok + kEE;
                U = dedup_tokens(ds, slots, E, m, false, &unused, lane, lo, hi);
                for (int x = lane; x < E; x += 32) lut[x] = (unsigned short)(lut[x] | slots[x]);
            }
            __syncwarp();
            for (int c0 = 0; c0 < c; c0 += kCG) {
                float acc[kT][2];
#pragma unroll
                for (int q = 0; q < kT; ++q) acc[q][0] = acc[q][1] = 0.f;
                for (int u0 = 0; u0 < U; u0 += kUR) {
                    const int Uc = min(kUR, U - u0);
                    __syncwarp();
                    // ---- dense weights of this pass: zero, then every entry whose merge row is in the pass
                    for (int z = lane; z < kT * kUR * ICT / 4; z += 32)
                        reinterpret_cast<float4*>(Wd)[z] = make_float4(0.f, 0.f, 0.f, 0.f);
                    __syncwarp();
#pragma unroll 2
                    for (int x = lane; x < E; x += 32) {
                        const unsigned lr = lut[x];
                        const int rel = (int)(lr & 0xfffu) - u0;
                        if (rel >= 0 && rel < Uc) {
                            const unsigned e = ent[x];
                            float w[ICT];
                            if (!(e & kDupFlag)) {
                                load_w<T, ICT>(Wb + (size_t)e * ICT, w);
                            } else {
                                // the merge row names the target several times: add its slots in order
                                const unsigned row = div_m(e & ~kDupFlag);
                                const int64_t* irow = idx_b + (long long)row * m;
#pragma unroll
                                for (int k = 0; k < ICT; ++k) w[k] = 0.f;
#pragma unroll 1
                                for (int j = 0; j < m; ++j)
                                    if (irow[j] == t0 + (int)(lr >> 12)) {
#pragma unroll
                                        for (int k = 0; k < ICT; ++k)
                                            w[k] += Elem<T>::up(Wb[((size_t)row * m + j) * ICT + k]);
                                    }
                            }
                            float* dst = Wd + ((lr >> 12) * kUR + rel) * ICT;
#pragma unroll
                            for (int k = 0; k < ICT; ++k) dst[k] = w[k];
                        }
                    }
                    __syncwarp();
                    // ---- the pass's merge rows, two in flight
                    auto fetch = [&](int u, float (&g)[ICT][2]) {
                        const T* gp = Gb + (long long)uniq[u0 + u] * (ICT * c) + c0;
#pragma unroll
                        for (int k = 0; k < ICT; ++k) {
                            if constexpr (std::is_same<T, float>::value) {
                                const float2 v = *reinterpret_cast<const float2*>(gp + k * c);
                                g[k][0] = v.x;  g[k][1] = v.y;
                            } else {
                                // two 16-bit channels in one word
                                const unsigned v = *reinterpret_cast<const unsigned*>(gp + k * c);
                                const unsigned short lo16 = (unsigned short)(v & 0xffffu), hi16 = (unsigned short)(v >> 16);
                                g[k][0] = Elem<T>::up(*reinterpret_cast<const T*>(&lo16));
                                g[k][1] = Elem<T>::up(*reinterpret_cast<const T*>(&hi16));
                            }
                        }
                    };
                    auto add = [&](int u, const float (&g)[ICT][2]) {
#pragma unroll
                        for (int q = 0; q < kT; ++q) {
                            float w[ICT];
                            const float* wp = Wd + (q * kUR + u) * ICT;
                            if constexpr (ICT == 4) {
                                const float4 v = *reinterpret_cast<const float4*>(wp);
                                w[0] = v.x;  w[1] = v.y;  w[2] = v.z;  w[3] = v.w;
                            } else if constexpr (ICT == 2) {
                                const float2 v = *reinterpret_cast<const float2*>(wp);
                                w[0] = v.x;  w[1] = v.y;
                            } else {
                                w[0] = wp[0];
                            }
#pragma unroll
                            for (int k = 0; k < ICT; ++k) {
                                acc[q][0] += w[k] * g[k][0];
                                acc[q][1] += w[k] * g[k][1];
                            }
                        }
                    };
                    float ga[ICT][2], gb[ICT][2];
                    int u = 0;
                    for (; u + 2 <= Uc; u += 2) {
                        fetch(u, ga);
                        fetch(u + 1, gb);
                        add(u, ga);
                        add(u + 1, gb);
                    }
                    if (u < Uc) {
                        fetch(u, ga);
                        add(u, ga);
                    }
                }
                // ---- the tile's outputs (added to what earlier chunks of a long entry list wrote)
#pragma unroll
                for (int q = 0; q < kT; ++q) {
                    if (t0 + q < n_tgt) {
                        T* dstp = Ob + (long long)(t0 + q) * c + c0;
                        float v0 = acc[q][0], v1 = acc[q][1];
                        if (e0 > 0) {
                            v0 += Elem<T>::up(dstp[0]);
                            v1 += Elem<T>::up(dstp[1]);
                        }
                        if constexpr (std::is_same<T, float>::value) {
                            *reinterpret_cast<float2*>(dstp) = make_float2(v0, v1);
                        } else {
                            const T a = Elem<T>::down(v0), bq = Elem<T>::down(v1);
                            const unsigned word = (unsigned)*reinterpret_cast<const unsigned short*>(&a) |
                                                  ((unsigned)*reinterpret_cast<const unsigned short*>(&bq) << 16);
                            *reinterpret_cast<unsigned*>(dstp) = word;
                        }
                    }
                }
            }
        }
    }
}

template <typename T, int ICT>
int wf_dfeat_rows_t(const char* label, const WfScatterParams& p, cudaStream_t s) {
    const size_t smem = size_t(kWarps) * WfRowsSmem::kTotal;
    auto kernel = p.m != kMmax ? wf_dfeat_rows_kernel<T, ICT, false, false>
                               : (p.c == kCG ? wf_dfeat_rows_kernel<T, ICT, true, true> : wf_dfeat_rows_kernel<T, ICT, true, false>);
    const int per_sm = resident_ctas(reinterpret_cast<const void*>(kernel), 32 * kWarps, smem);
    if (per_sm < 0) return per_sm;
    long long grid = (long long)sm_count() * per_sm;
    const long long need = ((long long)p.batch * p.tiles + kWarps - 1) / kWarps;
    if (grid > need) grid = need;
    ScopedKernelTimer timer(label, s);
    kernel<<<(int)grid, 32 * kWarps, smem, s>>>(p);
    note_launch();
    return check_launch();
}

template <typename T, int ICT>
int wf_dfeat_t(const char* label, const WfScatterParams& p, cudaStream_t s) {
    const size_t smem = size_t(kWarps) * WfScatterSmem::kTotal;
    auto kernel = p.m != kMmax ? wf_dfeat_kernel<T, ICT, false, false>
                               : (p.c == kCG ? wf_dfeat_kernel<T, ICT, true, true> : wf_dfeat_kernel<T, ICT, true, false>);
    const int per_sm = resident_ctas(reinterpret_cast<const void*>(kernel), 32 * kWarps, smem);
    if (per_sm < 0) return per_sm;
    long long grid = (long long)sm_count() * per_sm;
    const long long need = ((long long)p.batch * p.tiles + kWarps - 1) / kWarps;
    if (grid > need) grid = need;
    ScopedKernelTimer timer(label, s);
    kernel<<<(int)grid, 32 * kWarps, smem, s>>>(p);
    note_launch();
    return check_launch();
}

template <typename T>
int wf_dfeat_ic(const char* label, int ic, const WfScatterParams& p, cudaStream_t s) {
    // fp32: the unstaged kernel (0.290 -> 0.221 ms on the benchmark step); 16-bit inputs: the staged one, whose
    // products are single tensor-core instructions (0.221 against 0.226 ms).  CLUSTEN_WF_DFEAT = staged | rows
    // overrides the choice (read at every call).
    bool staged = !std::is_same<T, float>::value;
    if (const char* v = getenv("CLUSTEN_WF_DFEAT")) staged = v[0] == 's';
    switch (ic) {
        case 1: return staged ? wf_dfeat_t<T, 1>(label, p, s) : wf_dfeat_rows_t<T, 1>(label, p, s);
        case 2: return staged ? wf_dfeat_t<T, 2>(label, p, s) : wf_dfeat_rows_t<T, 2>(label, p, s);
        case 4: return staged ? wf_dfeat_t<T, 4>(label, p, s) : wf_dfeat_rows_t<T, 4>(label, p, s);
        default: return CLUSTEN_ERR_UNSUPPORTED;
    }
}

template <typename T, int MODE, int ICT>
int wf_tiles_t(const char* label, const WfParams& p, cudaStream_t s) {
    const size_t smem = size_t(kWarps) * WfSmem<MODE>::kTotal;
    auto kernel = p.m != kMmax ? wf_tiles_kernel<T, MODE, ICT, false, false>
                               : (p.c == kCG ? wf_tiles_kernel<T, MODE, ICT, true, true> : wf_tiles_kernel<T, MODE, ICT, true, false>);
    const int per_sm = resident_ctas(reinterpret_cast<const void*>(kernel), 32 * kWarps, smem);
    if (per_sm < 0) return per_sm;
    long long grid = (long long)sm_count() * per_sm;
    const long long need = ((long long)p.batch * p.tiles + kWarps - 1) / kWarps;
    if (grid > need) grid = need;
    ScopedKernelTimer timer(label, s);
    kernel<<<(int)grid, 32 * kWarps, smem, s>>>(p);
    note_launch();
    return check_launch();
}

template <typename T, int MODE>
int wf_tiles_ic(const char* label, int ic, const WfParams& p, cudaStream_t s) {
    switch (ic) {
        case 1: return wf_tiles_t<T, MODE, 1>(label, p, s);
        case 2: return wf_tiles_t<T, MODE, 2>(label, p, s);
        case 4: return wf_tiles_t<T, MODE, 4>(label, p, s);
        default: return CLUSTEN_ERR_UNSUPPORTED;
    }
}

template <int MODE>
int wf_tiles_dispatch(const char* label, int dtype, int ic, const WfParams& p, cudaStream_t s) {
    switch (dtype) {
        case CLUSTEN_F32: return wf_tiles_ic<float, MODE>(label, ic, p, s);
        case CLUSTEN_F16: return wf_tiles_ic<__half, MODE>(label, ic, p, s);
        case CLUSTEN_BF16: return wf_tiles_ic<__nv_bfloat16, MODE>(label, ic, p, s);
        default: return CLUSTEN_ERR_DTYPE;
    }
}

bool aligned16(std::initializer_list<const void*> ptrs) {
    for (const void* q : ptrs)
        if (reinterpret_cast<uintptr_t>(q) % 16 != 0) return false;
    return true;
}

}  // namespace

size_t wf_order_bytes(int b, int n_out) { return size_t(b) * n_out * sizeof(int); }

int launch_wf_order(const int64_t* idx, int b, int n_out, int m, int* order, cudaStream_t s) {
    if (n_out > kOrderMax) return CLUSTEN_ERR_UNSUPPORTED;
    ScopedKernelTimer timer("wf_order", s);
    wf_order_kernel<<<b, 1024, 0, s>>>(idx, order, n_out, m);
    note_launch();
    return check_launch();
}

bool tiled_wf_gather_supported(int dtype, const void* W, const void* F, const void* O, int n_out, int n, int m,
                               int ic, int c) {
    if (dtype != CLUSTEN_F32 && dtype != CLUSTEN_F16 && dtype != CLUSTEN_BF16) return false;
    if (c % kCG != 0 || (ic != 1 && ic != 2 && ic != 4) || m < 1 || m > kMmax || n > 65000 || n_out < 1) return false;
    if ((long long)n_out * m * ic > 0x7fffffffLL) return false;
    return aligned16({W, F, O});
}

int launch_tiled_wf_sum(const char* label, int dtype, const void* W, const void* F, const int64_t* idx,
                        const int* order, void* out, int b, int n_out, int n, int m, int ic, int c, cudaStream_t s) {
    if (wf_forward_direct_supported(dtype, n_out, n, m, ic, c) && getenv("CLUSTEN_WF_FORWARD_TILED") == nullptr)
        return launch_wf_forward_direct(label, dtype, W, F, idx, order, out, b, n_out, n, m, ic, c, s);
    WfParams p{};
    p.W = W;  p.F = F;  p.G = nullptr;  p.out = out;  p.idx = idx;  p.order = order;
    p.batch = b;  p.n_out = n_out;  p.n = n;  p.m = m;  p.c = c;  p.tiles = (n_out + kT - 1) / kT;
    if ((long long)b * p.tiles > 0x7fffffffLL) return CLUSTEN_ERR_SHAPE;
    return wf_tiles_dispatch<0>(label, dtype, ic, p, s);
}

bool tiled_wf_dfeat_supported(int dtype, const void* W, const void* G, const void* out, int n_out, int n, int m,
                              int ic, int c) {
    if (dtype != CLUSTEN_F32 && dtype != CLUSTEN_F16 && dtype != CLUSTEN_BF16) return false;
    if (c % kCG != 0 || (ic != 1 && ic != 2 && ic != 4) || m < 1 || n < 1 || n_out < 1 || n_out > 65000) return false;
    if ((long long)n_out * m * ic > 0x7fffffffLL) return false;
    return aligned16({W, G, out});
}

int launch_tiled_wf_dfeat(const char* label, int dtype, const void* W, const void* G, const int64_t* idx,
                          const InverseView& inv, void* d_feat, int b, int n_out, int n, int m, int ic, int c,
                          cudaStream_t s) {
    WfScatterParams p{};
    p.W = W;  p.G = G;  p.out = d_feat;  p.idx = idx;  p.inv = inv;
    p.batch = b;  p.n_out = n_out;  p.n = n;  p.m = m;  p.c = c;  p.tiles = (n + kT - 1) / kT;
    if ((long long)b * p.tiles > 0x7fffffffLL) return CLUSTEN_ERR_SHAPE;
    {   // x / m for x < 2^31:  (umulhi(magic, x) + x) >> shift
        unsigned l = 0;
        while ((1ull << l) < (unsigned)m) ++l;
        p.m_magic = (unsigned)(((1ull << 32) * ((1ull << l) - (unsigned)m)) / (unsigned)m + 1);
        p.m_shift = l;
    }
    switch (dtype) {
        case CLUSTEN_F32: return wf_dfeat_ic<float>(label, ic, p, s);
        case CLUSTEN_F16: return wf_dfeat_ic<__half>(label, ic, p, s);
        case CLUSTEN_BF16: return wf_dfeat_ic<__nv_bfloat16>(label, ic, p, s);
        default: return CLUSTEN_ERR_DTYPE;
    }
}

int launch_tiled_wf_dot(const char* label, int dtype, const void* F, const void* G, const int64_t* idx,
                        const int* order, void* d_weights, int b, int n_out, int n, int m, int ic, int c,
                        cudaStream_t s) {
    if (ic == 4 && dtype == CLUSTEN_F32 && wf_forward_direct_supported(dtype, n_out, n, m, ic, c) &&
        getenv("CLUSTEN_WF_DWEIGHTS_TILED") == nullptr)
        return launch_wf_dweights_direct(label, F, G, idx, order, d_weights, b, n_out, n, m, c, s);
    WfParams p{};
    p.W = nullptr;  p.F = F;  p.G = G;  p.out = d_weights;  p.idx = idx;  p.order = order;
    p.batch = b;  p.n_out = n_out;  p.n = n;  p.m = m;  p.c = c;  p.tiles = (n_out + kT - 1) / kT;
    if ((long long)b * p.tiles > 0x7fffffffLL) return CLUSTEN_ERR_SHAPE;
    return wf_tiles_dispatch<1>(label, dtype, ic, p, s);
}

}  // namespace clusten
