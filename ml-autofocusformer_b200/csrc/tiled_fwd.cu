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
constexpr int kOLD = 36;           // row stride (floats) of the output tile
constexpr int kYLD = 36;           // row stride (floats) of the fp32 Y tile
constexpr int kBMW = 256;          // bitmap words: token ids of a tile may span 8192
constexpr int kWarps = 4;          // warps per CTA (independent of each other)
constexpr int kEPL = kE / 32;      // edges per lane
constexpr unsigned kFull = 0xffffffffu;
constexpr unsigned short kSkip = 0xffffu;

// ----------------------------------------------------------------------------- shared memory (per warp)
//   X    neighbour rows [48][32] fp32; its front doubles as landing area of the tile's int64 indices
//   Xraw (16-bit inputs) the rows as loaded, converted to fp32 into X
//   Op   tiled_sum: weight tile [8][kWLD], later the output tile [8][kOLD];
//        tiled_dot: Y tile [8][kYLD] + score tile [8][kWLD];
//        doubles as bitmap scratch while a tile is de-duplicated
//   lut  edge -> slot,  uniq  slot -> source row
template <typename T, int MODE> struct WarpSmem {
    static constexpr bool kIsFloat = std::is_same<T, float>::value;
    static constexpr int kX = kUC * kC * 4;
    static constexpr int kXraw = kIsFloat ? 0 : kUC * kC * (int)sizeof(T);
    static constexpr int kOp = MODE == 0 ? kT * kWLD * 4 : (kT * kYLD + kT * kWLD) * 4;
    static constexpr int kLut = kE * 2;
    static constexpr int kTotal = kX + kXraw + kOp + 2 * kLut;
};
static_assert(kBMW * 4 + kBMW * 2 + (kE / 32) * 4 <= kT * kWLD * 4, "bitmap scratch must fit in Op");
static_assert(kT * kOLD <= kT * kWLD, "output tile must fit in Op");

// ----------------------------------------------------------------------------- PTX helpers
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16_ca(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(dst)), "l"(src));
}
__device__ __forceinline__ void cp_async16_cg(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(dst)), "l"(src));
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

// ----------------------------------------------------------------------------- products on the tensor cores
// mma.sync m16n8k8 with TF32 operands and FP32 accumulation.  FP32 inputs are split into a high
// part (upper 19 bits) and the exact remainder and multiplied in three passes (lo*hi, hi*lo,
// hi*hi), which keeps the result within a few 1e-7 of an FP32 product; FP16 / BF16 inputs are
// exactly representable in TF32, so one pass gives exact products.  Fragment layout (PTX ISA,
// m16n8k8): g = lane / 4, t = lane % 4;  A: a0=(g,t) a1=(g+8,t) a2=(g,t+4) a3=(g+8,t+4);
// B: b0=(t,g) b1=(t+4,g);  D: d0=(g,2t) d1=(g,2t+1) d2=(g+8,2t) d3=(g+8,2t+1).
__device__ __forceinline__ void mma_tf32(float (&d)[4], const unsigned (&a)[4], const unsigned (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void split_tf32(float x, unsigned& hi, unsigned& lo) {
    hi = __float_as_uint(x) & 0xffffe000u;
    lo = __float_as_uint(x - __uint_as_float(hi));
}
template <bool SPLIT, int NA>
__device__ __forceinline__ void mma_block(float (&d)[4], const float (&a)[4], const float (&b)[2]) {
    unsigned ah[4], bh[2];
    if (SPLIT) {
        unsigned al[4], bl[2];
#pragma unroll
        for (int i = 0; i < 4; ++i) split_tf32(a[i], ah[i], al[i]);
#pragma unroll
        for (int i = 0; i < 2; ++i) split_tf32(b[i], bh[i], bl[i]);
        mma_tf32(d, al, bh);
        mma_tf32(d, ah, bl);
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) ah[i] = __float_as_uint(a[i]);
#pragma unroll
        for (int i = 0; i < 2; ++i) bh[i] = __float_as_uint(b[i]);
    }
    mma_tf32(d, ah, bh);
}

// Fragment loads use 32-bit shared-memory addresses that are fixed per warp (computed once per kernel)
// plus compile-time offsets.
// Per-warp addresses for tiled_sum:  D[c][q] += sum_u Xs[u][c] * Wd[q][u].
// Xs rows are [32] floats with the 16-byte chunks of row r stored at chunk ^ ((r & 3) << 1); Wd has row
// stride kWLD.  With g = lane / 4, t = lane % 4 the B fragment comes from Wd row g, column u0 + t (+4) and
// the A fragment from staged row u0 + t (+4), channel 16 mt + 8 h + g.
struct SumAddr {
    unsigned w;          // &Wd[g][t]
    unsigned x[2][2];    // &Xs[t][16 mt + 8 h + g] (swizzled for rows with (row & 3) == t)
};
__device__ __forceinline__ SumAddr make_sum_addr(const float* Wd, const float* Xs, int lane) {
    const int g = lane >> 2, t = lane & 3;
    SumAddr a;
    a.w = smem_u32(Wd + g * kWLD + t);
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int c = 16 * mt + 8 * h + g;
            a.x[mt][h] = smem_u32(Xs + t * kC + ((((c >> 2) ^ (t << 1)) << 2) + (c & 3)));
        }
    return a;
}

#define CLUSTEN_LDS(dst, addr, off) asm volatile("ld.shared.f32 %0, [%1+" #off "];\n" : "=f"(dst) : "r"(addr))

template <int KS>
__device__ __forceinline__ void sum_load(const SumAddr& sa, float (&b)[2], float (&a)[2][4]) {
    // byte offsets: column / row u0 = 8 KS
    asm volatile("ld.shared.f32 %0, [%1+%2];\n" : "=f"(b[0]) : "r"(sa.w), "n"(KS * 8 * 4));
    asm volatile("ld.shared.f32 %0, [%1+%2];\n" : "=f"(b[1]) : "r"(sa.w), "n"((KS * 8 + 4) * 4));
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
        asm volatile("ld.shared.f32 %0, [%1+%2];\n" : "=f"(a[mt][0]) : "r"(sa.x[mt][0]), "n"(KS * 8 * kC * 4));
        asm volatile("ld.shared.f32 %0, [%1+%2];\n" : "=f"(a[mt][1]) : "r"(sa.x[mt][1]), "n"(KS * 8 * kC * 4));
        asm volatile("ld.shared.f32 %0, [%1+%2];\n" : "=f"(a[mt][2]) : "r"(sa.x[mt][0]), "n"((KS * 8 + 4) * kC * 4));
        asm volatile("ld.shared.f32 %0, [%1+%2];\n" : "=f"(a[mt][3]) : "r"(sa.x[mt][1]), "n"((KS * 8 + 4) * kC * 4));
    }
}

// All 48 staged rows: six steps, fully unrolled, operands of step k+1 fetched before step k multiplies.
template <bool SPLIT, int KS>
__device__ __forceinline__ void sum_steps48(const SumAddr& sa, float (&acc)[2][4], float (&b)[2], float (&a)[2][4]) {
    if constexpr (KS + 1 < kUC / 8) {
        float bn[2], an[2][4];
        sum_load<KS + 1>(sa, bn, an);
        mma_block<SPLIT, 0>(acc[0], a[0], b);
        mma_block<SPLIT, 0>(acc[1], a[1], b);
        sum_steps48<SPLIT, KS + 1>(sa, acc, bn, an);
    } else {
        mma_block<SPLIT, 0>(acc[0], a[0], b);
        mma_block<SPLIT, 0>(acc[1], a[1], b);
    }
}

template <bool SPLIT>
__device__ __forceinline__ void sum_product_mma(const SumAddr& sa, int rows8, float (&acc)[2][4]) {
    if (rows8 == kUC) {
        float b[2], a[2][4];
        sum_load<0>(sa, b, a);
        sum_steps48<SPLIT, 0>(sa, acc, b, a);
    } else {
        // partial chunk: one step at a time with running addresses
        SumAddr p = sa;
#pragma unroll 1
        for (int u0 = 0; u0 < rows8; u0 += 8) {
            float b[2], a[2][4];
            sum_load<0>(p, b, a);
            mma_block<SPLIT, 0>(acc[0], a[0], b);
            mma_block<SPLIT, 0>(acc[1], a[1], b);
            p.w += 8 * 4;
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
                p.x[mt][0] += 8 * kC * 4;
                p.x[mt][1] += 8 * kC * 4;
            }
        }
    }
}

// Per-warp addresses for tiled_dot:  Sb[q][u] = sum_c Xs[u][c] * Ys[q][c].
// Xs chunks of row r are stored at chunk ^ (r & 7); Ys has row stride kYLD; Sb row stride kWLD.
// A fragment: staged rows 16 mt + g (+8), channels k0 + t (+4);  B fragment: Ys row g, channels k0 + t (+4).
struct DotAddr {
    unsigned y;          // &Ys[g][t]
    unsigned x[8];       // &Xs[g][chunk c4 (swizzled with row & 7 == g)] + t
    unsigned s;          // &Sb[2 t][g]
};
__device__ __forceinline__ DotAddr make_dot_addr(const float* Ys, const float* Xs, const float* Sb, int lane) {
    const int g = lane >> 2, t = lane & 3;
    DotAddr a;
    a.y = smem_u32(Ys + g * kYLD + t);
#pragma unroll
    for (int c4 = 0; c4 < 8; ++c4) a.x[c4] = smem_u32(Xs + g * kC + ((c4 ^ g) << 2) + t);
    a.s = smem_u32(Sb + (2 * t) * kWLD + g);
    return a;
}

template <bool SPLIT, bool FULL>
__device__ __forceinline__ void dot_product_tiles(const DotAddr& da, int mtiles) {
    float acc[kUC / 16][4];
#pragma unroll
    for (int mt = 0; mt < kUC / 16; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < kC / 8; ++ks) {
        // channels 8 ks + t and 8 ks + 4 + t
        float bb[2];
        if (ks == 0) { CLUSTEN_LDS(bb[0], da.y, 0); CLUSTEN_LDS(bb[1], da.y, 16); }
        if (ks == 1) { CLUSTEN_LDS(bb[0], da.y, 32); CLUSTEN_LDS(bb[1], da.y, 48); }
        if (ks == 2) { CLUSTEN_LDS(bb[0], da.y, 64); CLUSTEN_LDS(bb[1], da.y, 80); }
        if (ks == 3) { CLUSTEN_LDS(bb[0], da.y, 96); CLUSTEN_LDS(bb[1], da.y, 112); }
#pragma unroll
        for (int mt = 0; mt < kUC / 16; ++mt) {
            if (FULL || mt < mtiles) {
                float a[4];
                // rows 16 mt + g and + 8: byte offsets 16 mt * 128 and + 8 * 128
                if (mt == 0) {
                    CLUSTEN_LDS(a[0], da.x[2 * ks], 0);     CLUSTEN_LDS(a[1], da.x[2 * ks], 1024);
                    CLUSTEN_LDS(a[2], da.x[2 * ks + 1], 0); CLUSTEN_LDS(a[3], da.x[2 * ks + 1], 1024);
                } else if (mt == 1) {
                    CLUSTEN_LDS(a[0], da.x[2 * ks], 2048);     CLUSTEN_LDS(a[1], da.x[2 * ks], 3072);
                    CLUSTEN_LDS(a[2], da.x[2 * ks + 1], 2048); CLUSTEN_LDS(a[3], da.x[2 * ks + 1], 3072);
                } else {
                    CLUSTEN_LDS(a[0], da.x[2 * ks], 4096);     CLUSTEN_LDS(a[1], da.x[2 * ks], 5120);
                    CLUSTEN_LDS(a[2], da.x[2 * ks + 1], 4096); CLUSTEN_LDS(a[3], da.x[2 * ks + 1], 5120);
                }
                mma_block<SPLIT, 0>(acc[mt], a, bb);
            }
        }
    }
    // D fragment -> Sb[q][u]: d0=(u=16mt+g, q=2t) d1=(u, 2t+1) d2=(u+8, 2t) d3=(u+8, 2t+1)
#pragma unroll
    for (int mt = 0; mt < kUC / 16; ++mt) {
        if (FULL || mt < mtiles) {
            if (mt == 0) {
                asm volatile("st.shared.f32 [%0+0], %1;\n" ::"r"(da.s), "f"(acc[0][0]));
                asm volatile("st.shared.f32 [%0+208], %1;\n" ::"r"(da.s), "f"(acc[0][1]));
                asm volatile("st.shared.f32 [%0+32], %1;\n" ::"r"(da.s), "f"(acc[0][2]));
                asm volatile("st.shared.f32 [%0+240], %1;\n" ::"r"(da.s), "f"(acc[0][3]));
            } else if (mt == 1) {
                asm volatile("st.shared.f32 [%0+64], %1;\n" ::"r"(da.s), "f"(acc[1][0]));
                asm volatile("st.shared.f32 [%0+272], %1;\n" ::"r"(da.s), "f"(acc[1][1]));
                asm volatile("st.shared.f32 [%0+96], %1;\n" ::"r"(da.s), "f"(acc[1][2]));
                asm volatile("st.shared.f32 [%0+304], %1;\n" ::"r"(da.s), "f"(acc[1][3]));
            } else {
                asm volatile("st.shared.f32 [%0+128], %1;\n" ::"r"(da.s), "f"(acc[2][0]));
                asm volatile("st.shared.f32 [%0+336], %1;\n" ::"r"(da.s), "f"(acc[2][1]));
                asm volatile("st.shared.f32 [%0+160], %1;\n" ::"r"(da.s), "f"(acc[2][2]));
                asm volatile("st.shared.f32 [%0+368], %1;\n" ::"r"(da.s), "f"(acc[2][3]));
            }
        }
    }
}
static_assert(kWLD * 4 == 208 && kC * 4 == 128 && kUC == 48, "byte offsets above are written out for these sizes");

template <bool SPLIT>
__device__ __forceinline__ void dot_product_mma(const DotAddr& da, int mtiles) {
    if (mtiles == kUC / 16) dot_product_tiles<SPLIT, true>(da, mtiles);
    else dot_product_tiles<SPLIT, false>(da, mtiles);
}

// ----------------------------------------------------------------------------- producer: tile analysis
// Are the 8 rows of the tile identical, in range, and the tile complete?  One warp.
// col0 = (2 * lane) % m and col_step = 64 % m are the column of the lane's first entry pair and its
// advance per pass (computed once per kernel).
__device__ __forceinline__ bool rows_identical(const long long* ring, int E, int m, int n, bool complete,
                                               int lane, int col0, int col_step) {
    const int4* r = reinterpret_cast<const int4*>(ring) + lane;      // {lo, hi, lo, hi} of two entries
    const int4* r0 = reinterpret_cast<const int4*>(ring);
    bool same = complete && (m & 7) == 0;
    int col = col0;
#pragma unroll
    for (int k = 0; k < kE / 64; ++k) {
        if (2 * (lane + 32 * k) < E) {
            const int4 v = r[32 * k];
            const int4 ref = r0[col >> 1];
            if (v.x != ref.x || v.z != ref.z || (v.y | v.w) != 0 || (unsigned)v.x >= (unsigned)n ||
                (unsigned)v.z >= (unsigned)n)
                same = false;
            col += col_step;
            if (col >= m) col -= m;
        }
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
__device__ int dedup_tokens(const DedupScratch ps_, unsigned short* lut, int E, int m, bool want_rowdup,
                            bool* rowdup, int lane, int lo, int hi);

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
    return dedup_tokens(ps_, lut, E, m, want_rowdup, rowdup, lane, lo, hi);
}

// ps.tok[0..E) (kSkip = none) with its value range [lo, hi] over the lanes -> lut, ps.uniq; returns U.
__device__ int dedup_tokens(const DedupScratch ps_, unsigned short* lut, int E, int m, bool want_rowdup,
                            bool* rowdup, int lane, int lo, int hi) {
    const DedupScratch* ps = &ps_;
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

    int* tok_s = reinterpret_cast<int*>(uniq);                        // identical rows: source row of X row r
    const SumAddr sa = make_sum_addr(Wd, Xs, lane);                   // MODE 0
    const DotAddr da = make_dot_addr(Ys, Xs, Sb, lane);               // MODE 1

    const int E = kT * m;
    const int m4 = m >> 2;
    // word offset of 16-byte chunk ci inside staged row r = qi + 4k (k even / odd):
    // tiled_sum stores chunk ^ ((r & 3) << 1), tiled_dot chunk ^ (r & 7), see the product routines
    const int sw_even = MODE == 0 ? ((ci ^ (qi << 1)) << 2) : ((ci ^ qi) << 2);
    const int sw_odd = MODE == 0 ? sw_even : (sw_even ^ 16);
    // piece z = lane + 32k of a [8][m] tile -> (row, 4-element piece); edge x = lane + 32k -> its row
    int wq[3], wc[3];
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        const int z = lane + 32 * k;
        const int d = m4 > 0 ? m4 : 1;
        wq[k] = z / d;
        wc[k] = z - wq[k] * d;
    }
    const int col0 = (2 * lane) % m, col_step = 64 % m;
    unsigned long long qpack = 0ull;                    // 3 bits per edge: its row
#pragma unroll
    for (int k = 0; k < kEPL; ++k) qpack |= (unsigned long long)(((lane + 32 * k) / m) & 7) << (3 * k);

    const unsigned total = (unsigned)batch * (unsigned)tiles;       // < 2^31, checked by the launcher
    const unsigned nwarps = gridDim.x * kWarps;
    const unsigned task0 = blockIdx.x * kWarps + warp;
    int b = (int)(task0 / (unsigned)tiles);
    int tile = (int)(task0 - (unsigned)b * (unsigned)tiles);
    const int step_b = (int)(nwarps / (unsigned)tiles), step_t = (int)(nwarps % (unsigned)tiles);
    int nb = b + step_b, ntile = tile + step_t;                      // this warp's next (batch, tile)
    if (ntile >= tiles) { ntile -= tiles; ++nb; }
    for (unsigned task = task0; task < total; task += nwarps) {
        const int i0 = tile * kT;
        const bool complete = i0 + kT <= n;
        const int64_t* src = idx + ((long long)b * n + i0) * m;
        // ---- warm the L2 for this warp's next tile: its index rows and its weight / Y rows
        {
            if (nb < batch) {
                const int ni0 = ntile * kT;
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
        const bool identical = rows_identical(ring, E, m, n, complete, lane, col0, col_step);
        int U = m;
        bool rowdup = false;
        if (identical) {
            const int* ring32 = reinterpret_cast<const int*>(ring);
            for (int r = lane; r < m; r += 32) tok_s[r] = ring32[2 * r];
        } else {
            U = dedup_tile(ds, ring, lut, E, m, i0, n, MODE == 0, &rowdup, lane);
        }
        __syncwarp();                                    // the landing area is free again

        for (int g = 0; g < heads; ++g) {
            const long long bb = (long long)b * heads + g;
            const T* Xh = X + (bb * n) * kC;
            float acc[2][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[0][i] = acc[1][i] = 0.f;
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
                if (kIsFloat && identical) {
                    const T* Xl = Xh + ci * 4;
                    float* dst = Xs + qi * kC;
#pragma unroll
                    for (int k = 0; k < kUC / 4; ++k)
                        if (qi + 4 * k < m)
                            cp_async16_cg(dst + 4 * k * kC + ((k & 1) ? sw_odd : sw_even), Xl + (long long)tok_s[qi + 4 * k] * kC);
                } else if (kIsFloat) {
#pragma unroll
                    for (int k = 0; k < kUC / 4; ++k) {
                        const int r = qi + 4 * k;
                        if (r < rows8) {
                            int t = -1;
                            if (r < Uc) {
                                if (identical) t = tok_s[r];
                                else {
                                    const unsigned short tt = uniq[u0 + r];
                                    t = tt == kSkip ? -1 : (int)tt;
                                }
                            }
                            float* dst = Xs + r * kC + ((k & 1) ? sw_odd : sw_even);
                            if (t >= 0) cp_async16_cg(dst, Xh + (long long)t * kC + ci * 4);
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
                                if (identical) t = tok_s[r];
                                else {
                                    const unsigned short tt = uniq[u0 + r];
                                    t = tt == kSkip ? -1 : (int)tt;
                                }
                            }
                            T* dst = Xraw + r * kC + pc * kPer;
                            if (t >= 0) cp_async16_cg(dst, Xh + (long long)t * kC + pc * kPer);
                            else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                    }
                }
                if (MODE == 0) {
                    // ---- weight tile -> Wd while the rows are on their way
                    const T* Wt = A + (bb * n + i0) * m;
                    if (identical) {
#pragma unroll
                        for (int k = 0; k < 3; ++k)
                            if (lane + 32 * k < kT * m4) {
                                float* dd = Wd + wq[k] * kWLD + wc[k] * 4;
                                if (kIsFloat) cp_async16_ca(dd, Wt + wq[k] * m + wc[k] * 4);
                                else *reinterpret_cast<float4*>(dd) = ld4(Wt + wq[k] * m + wc[k] * 4);
                            }
                    } else {
                        for (int z = lane; z < kT * kWLD / 4; z += 32)
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
                                        Wd[q * kWLD + rel] = w;
                                    }
                                }
                            }
                        } else if (lane < kT) {
                            // some row repeats a neighbour: one lane per row adds the weights in column order
                            for (int j = 0; j < m; ++j) {
                                const unsigned short sl = lut[lane * m + j];
                                const int rel = (int)sl - u0;
                                if (sl != kSkip && rel >= 0 && rel < Uc) {
                                    Wd[lane * kWLD + rel] += Elem<T>::up(Wt[lane * m + j]);
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
                cp_async_commit();
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
                    sum_product_mma<kIsFloat>(sa, rows8, acc);
                } else {
                    dot_product_mma<kIsFloat>(da, (Uc + 15) >> 4);
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
                // D fragments -> output tile [8][kOLD] in shared memory -> 16-byte stores
                float* Ot = Op;
                const int g = lane >> 2, t = lane & 3;
                __syncwarp();
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    float* o = Ot + (2 * t) * kOLD + 16 * mt + g;
                    o[0] = acc[mt][0];
                    o[kOLD] = acc[mt][1];
                    o[8] = acc[mt][2];
                    o[kOLD + 8] = acc[mt][3];
                }
                __syncwarp();
#pragma unroll
                for (int a = 0; a < 2; ++a) {
                    const int q = 2 * qi + a;
                    if (i0 + q < n)
                        st4(out + (bb * n + i0 + q) * kC + ci * 4,
                            *reinterpret_cast<const float4*>(Ot + q * kOLD + ci * 4));
                }
            }
        }
        // advance to this warp's next (batch, tile)
        b = nb;
        tile = ntile;
        nb += step_b;
        ntile += step_t;
        if (ntile >= tiles) {
            ntile -= tiles;
            ++nb;
        }
    }
}

// ----------------------------------------------------------------------------- scatter side (d_key, d_value, d_feat)
//   out[b, t, 32 s .. 32 s + 31] = sum over inverse-index entries (i, j) of target t and k < ic:
//                                   W[b, s, (i * m + j) * ic + k] * X[b, s, i * ic + k, :]
// Same scheme with targets as tile rows: a warp takes 8 consecutive targets, concatenates their
// inverse-index segments (512 edges at a time), de-duplicates the SOURCE rows, stages each once per
// 32-channel slab ("head") and multiplies the dense [8 x U] weights on the tensor cores.  Segments
// are ordered by source row and slots ascend with the source row, so the summation order is fixed.
// QK / AV: ic = 1, a slab is a head.  WF: a slab is 32 of the c channels, the weights are shared by
// the slabs and every entry fans out into its ic (weight, row) pairs.
struct ScatterParams {
    const void* W;  long long w_batch, w_head;                 // element strides
    const void* X;  long long x_batch, x_head;  int x_row;
    void* out;      long long o_batch, o_head;  int o_row;
    const int64_t* idx;  int idx_rows;  int m;                   // nbhd_idx [batch][idx_rows][m]
    InverseView inv;  int n_tgt;
    int ic, heads, batch, tiles;
    unsigned m_magic, m_shift, ic_magic, ic_shift;              // x / d = (umulhi(magic, x) + x) >> shift
};
__device__ __forceinline__ unsigned fast_div(unsigned x, unsigned magic, unsigned shift) {
    return (__umulhi(magic, x) + x) >> shift;
}

constexpr int kES = 512;            // edges handled at a time (8 targets x ~48 on average)

template <typename T> struct ScatterSmem {
    static constexpr bool kIsFloat = std::is_same<T, float>::value;
    static constexpr int kX = kUC * kC * 4;         // staged rows; de-duplication scratch before that
    static constexpr int kXraw = kIsFloat ? 0 : kUC * kC * (int)sizeof(T);
    static constexpr int kOp = kT * kWLD * 4;       // dense weights; bitmap scratch; output tile
    static constexpr int kEdge = kES * 4;           // weight index of each edge (bit 31: target repeats in its row)
    static constexpr int kWbuf = kES * 4;           // weight of each edge for the current slab
    static constexpr int kLut = kES * 2;            // slot | tile row << 12;   slot -> source row
    static constexpr int kTotal = kX + kXraw + kOp + kEdge + kWbuf + 2 * kLut;
};
static_assert(2 * kES * 2 <= kUC * kC * 4, "token and slot scratch must fit in the row buffer");

template <typename T>
__global__ void __launch_bounds__(32 * kWarps, 4)
scatter_tiles_kernel(const ScatterParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    using WS = ScatterSmem<T>;
    constexpr bool kIsFloat = WS::kIsFloat;
    constexpr int kPer = 16 / (int)sizeof(T);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int qi = lane >> 3, ci = lane & 7;
    unsigned char* base = smem_raw + size_t(warp) * WS::kTotal;
    float* Xs = reinterpret_cast<float*>(base);
    T* Xraw = reinterpret_cast<T*>(base + WS::kX);
    float* Wd = reinterpret_cast<float*>(base + WS::kX + WS::kXraw);
    unsigned* edge = reinterpret_cast<unsigned*>(base + WS::kX + WS::kXraw + WS::kOp);
    float* wbuf = reinterpret_cast<float*>(base + WS::kX + WS::kXraw + WS::kOp + WS::kEdge);
    unsigned short* lut = reinterpret_cast<unsigned short*>(base + WS::kX + WS::kXraw + WS::kOp + WS::kEdge + WS::kWbuf);
    unsigned short* uniq = lut + kES;
    DedupScratch ds;
    ds.tok = reinterpret_cast<unsigned short*>(base);           // the row buffer is free while de-duplicating
    unsigned short* slots = ds.tok + kES;
    ds.uniq = uniq;
    ds.bm = reinterpret_cast<unsigned*>(Wd);
    ds.pre = reinterpret_cast<unsigned short*>(ds.bm + kBMW);
    ds.rowbm = reinterpret_cast<unsigned*>(ds.pre + kBMW);
    const SumAddr sa = make_sum_addr(Wd, Xs, lane);
    const int sw = (ci ^ (qi << 1)) << 2;                       // chunk swizzle of staged row qi + 4k
    const int m = p.m, ic = p.ic, n_tgt = p.n_tgt;
    const T* Wg = static_cast<const T*>(p.W);
    const T* Xg = static_cast<const T*>(p.X);
    T* Og = static_cast<T*>(p.out);

    const unsigned total = (unsigned)p.batch * (unsigned)p.tiles;
    const unsigned nwarps = gridDim.x * kWarps;
    // segment (length, start) of target t0 + lane of a task, lanes 0..7
    auto load_segment = [&](unsigned task, int& len, int& start) {
        len = 0;
        start = 0;
        if (task < total) {
            const int b = (int)(task / (unsigned)p.tiles);
            const int t = (int)(task - (unsigned)b * (unsigned)p.tiles) * kT + lane;
            if (lane < kT && t < n_tgt) {
                len = p.inv.seglen[(long long)b * n_tgt + t];
                start = p.inv.rowptr[(long long)b * (n_tgt + 1) + t];
            }
        }
    };
    int next_len, next_start;
    load_segment(blockIdx.x * kWarps + warp, next_len, next_start);
    for (unsigned task = blockIdx.x * kWarps + warp; task < total; task += nwarps) {
        const int b = (int)(task / (unsigned)p.tiles);
        const int t0 = (int)(task - (unsigned)b * (unsigned)p.tiles) * kT;
        const int64_t* idx_b = p.idx + (long long)b * p.idx_rows * m;
        const int* entries = p.inv.entries + (long long)b * p.idx_rows * m;
        const int len = next_len * ic, start = next_start;      // every entry fans out into ic edges
        load_segment(task + nwarps, next_len, next_start);      // in flight while this tile is worked on
        int incl = len;
#pragma unroll
        for (int o = 1; o < kT; o <<= 1) {
            const int y = __shfl_up_sync(kFull, incl, o);
            if (lane >= o) incl += y;
        }
        const int E_total = __shfl_sync(kFull, incl, kT - 1);
        int off[kT], st[kT];                                    // per tile row: offset in the edge list, segment start
#pragma unroll
        for (int r = 0; r < kT; ++r) {
            off[r] = __shfl_sync(kFull, incl - len, r);
            st[r] = __shfl_sync(kFull, start, r);
        }

        for (int e0 = 0; e0 == 0 || e0 < E_total; e0 += kES) {
            const int E = max(0, min(kES, E_total - e0));
            // ---- this chunk's edges: weight index (flagged when the target repeats in its row), source
            //      row, tile row
            int lo = INT_MAX, hi = -1;
            bool any_flag = false;
            __syncwarp();
#pragma unroll 4
            for (int x = lane; x < E; x += 32) {
                const int pe = e0 + x;
                int r = 0;
#pragma unroll
                for (int j = 1; j < kT; ++j) r += (pe >= off[j]) ? 1 : 0;
                int s0 = st[0], o0 = off[0];
#pragma unroll
                for (int j = 1; j < kT; ++j)
                    if (r == j) {
                        s0 = st[j];
                        o0 = off[j];
                    }
                const unsigned q = (unsigned)(pe - o0);                     // position inside the fanned-out segment
                const unsigned qe = fast_div(q, p.ic_magic, p.ic_shift);     // entry inside the segment
                const unsigned k = q - qe * (unsigned)ic;
                const unsigned e = (unsigned)__ldg(entries + s0 + (int)qe);
                const unsigned plain = e & ~kDupFlag;                       // row * m + slot
                const unsigned src = fast_div(plain, p.m_magic, p.m_shift);
                edge[x] = (plain * (unsigned)ic + k) | (e & kDupFlag);
                const int srow = (int)(src * (unsigned)ic + k);
                ds.tok[x] = (unsigned short)srow;
                lut[x] = (unsigned short)(r << 12);                         // the slot is merged in below
                lo = min(lo, srow);
                hi = max(hi, srow);
                if (e & kDupFlag) any_flag = true;
            }
            any_flag = __any_sync(kFull, any_flag);
            int U = 0;
            if (E > 0) {
                bool unused = false;
                U = dedup_tokens(ds, slots, E, m, false, &unused, lane, lo, hi);
                for (int x = lane; x < E; x += 32) lut[x] = (unsigned short)(lut[x] | slots[x]);
            }
            __syncwarp();

            for (int g = 0; g < p.heads; ++g) {
                const T* Wh = Wg + (long long)b * p.w_batch + (long long)g * p.w_head;
                const T* Xh = Xg + (long long)b * p.x_batch + (long long)g * p.x_head;
                // ---- weights of the edges for this slab
                if (g == 0 || p.w_head != 0) {
#pragma unroll 4
                    for (int x = lane; x < E; x += 32) {
                        const unsigned e = edge[x];
                        wbuf[x] = (e & kDupFlag) ? 0.f : Elem<T>::up(Wh[e]);
                    }
                    if (any_flag) {
                        // targets that occur several times in their source row: sum that row's slots in order
                        for (int x = lane; x < E; x += 32) {
                            const unsigned e = edge[x];
                            if (e & kDupFlag) {
                                const unsigned we = e & ~kDupFlag;
                                const unsigned pl = fast_div(we, p.ic_magic, p.ic_shift);
                                const unsigned k = we - pl * (unsigned)ic;
                                const unsigned row = fast_div(pl, p.m_magic, p.m_shift);
                                const int t = t0 + (lut[x] >> 12);
                                const int64_t* irow = idx_b + (long long)row * m;
                                float w = 0.f;
                                for (int j = 0; j < m; ++j)
                                    if (irow[j] == t) w += Elem<T>::up(Wh[((long long)row * m + j) * ic + k]);
                                wbuf[x] = w;
                            }
                        }
                    }
                }
                float acc[2][4];
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[0][i] = acc[1][i] = 0.f;
                for (int u0 = 0; u0 < U; u0 += kUC) {
                    const int Uc = min(kUC, U - u0);
                    const int rows8 = (Uc + 7) & ~7;
                    __syncwarp();
                    if (kIsFloat) {
#pragma unroll
                        for (int k = 0; k < kUC / 4; ++k) {
                            const int r = qi + 4 * k;
                            if (r < rows8) {
                                float* dst = Xs + r * kC + sw;
                                if (r < Uc) cp_async16_cg(dst, Xh + (long long)uniq[u0 + r] * p.x_row + ci * 4);
                                else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
                            }
                        }
                    } else {
                        const int pr = lane >> 2, pc = lane & 3;
#pragma unroll
                        for (int k = 0; k < kUC / 8; ++k) {
                            const int r = pr + 8 * k;
                            if (r < rows8) {
                                T* dst = Xraw + r * kC + pc * kPer;
                                if (r < Uc) cp_async16_cg(dst, Xh + (long long)uniq[u0 + r] * p.x_row + pc * kPer);
                                else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
                            }
                        }
                    }
                    cp_async_commit();
                    for (int z = lane; z < kT * kWLD / 4; z += 32)
                        reinterpret_cast<float4*>(Wd)[z] = make_float4(0.f, 0.f, 0.f, 0.f);
                    __syncwarp();
#pragma unroll 4
                    for (int x = lane; x < E; x += 32) {
                        const unsigned lr = lut[x];
                        const int rel = (int)(lr & 0xfffu) - u0;
                        if (rel >= 0 && rel < Uc) Wd[(lr >> 12) * kWLD + rel] = wbuf[x];
                    }
                    cp_async_wait<0>();
                    __syncwarp();
                    if (!kIsFloat) {
#pragma unroll
                        for (int k = 0; k < kUC / 4; ++k) {
                            const int r = qi + 4 * k;
                            if (r < rows8) st4(Xs + r * kC + sw, ld4(Xraw + r * kC + ci * 4));
                        }
                        __syncwarp();
                    }
                    sum_product_mma<kIsFloat>(sa, rows8, acc);
                }
                // D fragments -> output tile in shared memory -> 16-byte stores (added to what earlier
                // chunks of a long edge list wrote)
                float* Ot = Wd;
                const int gg = lane >> 2, tt = lane & 3;
                __syncwarp();
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    float* o = Ot + (2 * tt) * kOLD + 16 * mt + gg;
                    o[0] = acc[mt][0];
                    o[kOLD] = acc[mt][1];
                    o[8] = acc[mt][2];
                    o[kOLD + 8] = acc[mt][3];
                }
                __syncwarp();
                T* Oh = Og + (long long)b * p.o_batch + (long long)g * p.o_head;
#pragma unroll
                for (int a = 0; a < 2; ++a) {
                    const int q = 2 * qi + a;
                    if (t0 + q < n_tgt) {
                        T* dstp = Oh + (long long)(t0 + q) * p.o_row + ci * 4;
                        float4 v = *reinterpret_cast<const float4*>(Ot + q * kOLD + ci * 4);
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
    if ((long long)b * tiles > 0x7fffffffLL) return CLUSTEN_ERR_SHAPE;
    const size_t smem = size_t(kWarps) * WarpSmem<T, MODE>::kTotal;
    auto kernel = gather_tiles_kernel<T, MODE>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return CLUSTEN_ERR_CUDA;
    }
    // one resident wave of CTAs; every warp strides over the (batch, tile) pairs
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 32 * kWarps, smem) != cudaSuccess) {
        cudaGetLastError();
        return CLUSTEN_ERR_CUDA;
    }
    long long grid = (long long)sm_count() * (per_sm > 0 ? per_sm : 1);
    const long long need = ((long long)b * tiles + kWarps - 1) / kWarps;
    if (grid > need) grid = need;
    ScopedKernelTimer timer(label, s);
    kernel<<<(int)grid, 32 * kWarps, smem, s>>>((const T*)A, (const T*)X, idx, (T*)out, b, h, n, m, tiles);
    note_launch();
    return check_launch();
}

// magic numbers for x / d with x < 2^31: q = (umulhi(magic, x) + x) >> shift
void div_magic(unsigned d, unsigned* magic, unsigned* shift) {
    unsigned l = 0;
    while ((1ull << l) < d) ++l;
    *magic = (unsigned)(((1ull << 32) * ((1ull << l) - d)) / d + 1);
    *shift = l;
}

template <typename T>
int scatter_tiles_t(const char* label, ScatterParams p, cudaStream_t s) {
    p.tiles = (p.n_tgt + kT - 1) / kT;
    if ((long long)p.batch * p.tiles > 0x7fffffffLL) return CLUSTEN_ERR_SHAPE;
    div_magic((unsigned)p.m, &p.m_magic, &p.m_shift);
    div_magic((unsigned)p.ic, &p.ic_magic, &p.ic_shift);
    const size_t smem = size_t(kWarps) * ScatterSmem<T>::kTotal;
    auto kernel = scatter_tiles_kernel<T>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return CLUSTEN_ERR_CUDA;
    }
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 32 * kWarps, smem) != cudaSuccess) {
        cudaGetLastError();
        return CLUSTEN_ERR_CUDA;
    }
    long long grid = (long long)sm_count() * (per_sm > 0 ? per_sm : 1);
    const long long need = ((long long)p.batch * p.tiles + kWarps - 1) / kWarps;
    if (grid > need) grid = need;
    ScopedKernelTimer timer(label, s);
    kernel<<<(int)grid, 32 * kWarps, smem, s>>>(p);
    note_launch();
    return check_launch();
}

int scatter_dispatch(const char* label, int dtype, const ScatterParams& p, cudaStream_t s) {
    switch (dtype) {
        case CLUSTEN_F32: return scatter_tiles_t<float>(label, p, s);
        case CLUSTEN_F16: return scatter_tiles_t<__half>(label, p, s);
        case CLUSTEN_BF16: return scatter_tiles_t<__nv_bfloat16>(label, p, s);
        default: return CLUSTEN_ERR_DTYPE;
    }
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

namespace clusten {

bool tiled_scatter_supported(int dtype, const void* W, const void* X, const void* out, int n, int m, int c) {
    return gather_supported(dtype, {X, out}, n, 1, c) && m >= 1 && reinterpret_cast<uintptr_t>(W) % 4 == 0;
}
int launch_tiled_scatter(const char* label, int dtype, const void* W, const void* X, const int64_t* idx,
                         const InverseView& inv, void* out, int b, int h, int n, int m, cudaStream_t s) {
    ScatterParams p{};
    p.W = W;  p.w_batch = (long long)h * n * m;  p.w_head = (long long)n * m;
    p.X = X;  p.x_batch = (long long)h * n * kC; p.x_head = (long long)n * kC;  p.x_row = kC;
    p.out = out;  p.o_batch = p.x_batch;  p.o_head = p.x_head;  p.o_row = kC;
    p.idx = idx;  p.idx_rows = n;  p.m = m;  p.inv = inv;  p.n_tgt = n;
    p.ic = 1;  p.heads = h;  p.batch = b;
    return scatter_dispatch(label, dtype, p, s);
}

// WF: d_feat[b, t, :] over c channels in slabs of 32; rows of X are d_feat_new[b, i, k, :]
bool tiled_wf_scatter_supported(int dtype, const void* W, const void* X, const void* out, int n_out, int n, int m,
                                int ic, int c) {
    if (dtype != CLUSTEN_F32 && dtype != CLUSTEN_F16 && dtype != CLUSTEN_BF16) return false;
    if (c % kC != 0 || ic < 1 || ic > 16 || m < 1 || n < 1 || (long long)n_out * ic > 65000) return false;
    return reinterpret_cast<uintptr_t>(X) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0 &&
           reinterpret_cast<uintptr_t>(W) % 4 == 0;
}
int launch_tiled_wf_scatter(const char* label, int dtype, const void* W, const void* X, const int64_t* idx,
                            const InverseView& inv, void* out, int b, int n_out, int n, int m, int ic, int c,
                            cudaStream_t s) {
    ScatterParams p{};
    p.W = W;  p.w_batch = (long long)n_out * m * ic;  p.w_head = 0;
    p.X = X;  p.x_batch = (long long)n_out * ic * c;  p.x_head = kC;  p.x_row = c;
    p.out = out;  p.o_batch = (long long)n * c;  p.o_head = kC;  p.o_row = c;
    p.idx = idx;  p.idx_rows = n_out;  p.m = m;  p.inv = inv;  p.n_tgt = n;
    p.ic = ic;  p.heads = c / kC;  p.batch = b;
    return scatter_dispatch(label, dtype, p, s);
}

}  // namespace clusten
