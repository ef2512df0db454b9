// Building blocks of the tiled CLUSTEN kernels: constants, cp.async / conversion helpers, the
// tensor-core products on staged neighbour rows and the warp-level de-duplication of a tile's indices.
// Included by tiled_fwd.cu (QK / AV gather and scatter side) and wf_tiled.cu (the WF kernels); every
// definition has internal linkage.
#pragma once

#include <limits.h>
#include <type_traits>

#include "tiled.cuh"

namespace clusten {
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
constexpr int kDirectU = 144;      // more distinct neighbour rows than this in a tile: gather them unstaged
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
__device__ __forceinline__ void cp_async4_ca(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_u32(dst)), "l"(src));
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

// Two accumulators fed by the same B fragment: the passes of the two products alternate, so that an MMA
// never directly follows the one whose accumulator it reads.
template <bool SPLIT>
__device__ __forceinline__ void mma_pair(float (&d)[2][4], const float (&a)[2][4], const float (&b)[2]) {
    unsigned ah[2][4], bh[2];
    if (SPLIT) {
        unsigned al[2][4], bl[2];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) split_tf32(a[mt][i], ah[mt][i], al[mt][i]);
#pragma unroll
        for (int i = 0; i < 2; ++i) split_tf32(b[i], bh[i], bl[i]);
        mma_tf32(d[0], al[0], bh);
        mma_tf32(d[1], al[1], bh);
        mma_tf32(d[0], ah[0], bl);
        mma_tf32(d[1], ah[1], bl);
    } else {
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) ah[mt][i] = __float_as_uint(a[mt][i]);
#pragma unroll
        for (int i = 0; i < 2; ++i) bh[i] = __float_as_uint(b[i]);
    }
    mma_tf32(d[0], ah[0], bh);
    mma_tf32(d[1], ah[1], bh);
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
        mma_pair<SPLIT>(acc, a, b);
        sum_steps48<SPLIT, KS + 1>(sa, acc, bn, an);
    } else {
        mma_pair<SPLIT>(acc, a, b);
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
            mma_pair<SPLIT>(acc, a, b);
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
        unsigned bh[2], bl[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            if (SPLIT) split_tf32(bb[i], bh[i], bl[i]);
            else { bh[i] = __float_as_uint(bb[i]); bl[i] = 0u; }
        }
        unsigned ah[kUC / 16][4];
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
                // the low-part pass of a row tile goes out as soon as its operands are there; the other two
                // passes follow tile by tile below, so consecutive MMAs never share an accumulator
                unsigned al[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (SPLIT) split_tf32(a[i], ah[mt][i], al[i]);
                    else ah[mt][i] = __float_as_uint(a[i]);
                }
                if (SPLIT) mma_tf32(acc[mt], al, bh);
            }
        }
        if (SPLIT) {
#pragma unroll
            for (int mt = 0; mt < kUC / 16; ++mt)
                if (FULL || mt < mtiles) mma_tf32(acc[mt], ah[mt], bl);
        }
#pragma unroll
        for (int mt = 0; mt < kUC / 16; ++mt)
            if (FULL || mt < mtiles) mma_tf32(acc[mt], ah[mt], bh);
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

// ----------------------------------------------------------------------------- 16-bit products
// FP16 / BF16 inputs stay 16-bit in shared memory and are multiplied with mma.sync m16n8k16 (FP32
// accumulation, exact products).  Staged rows are [row][32 elements] = 64 bytes; the 16-byte chunk c of
// row r is stored at chunk c ^ ((r >> 1) & 3), which makes the 8-row ldmatrix accesses conflict free.
// Fragment layout (PTX ISA, m16n8k16): A regs a0=(g, 2t..2t+1) a1=(g+8, ..) a2=(g, 2t+8..) a3=(g+8, 2t+8..);
// B regs b0=(k=2t..2t+1, n=g) b1=(k=2t+8.., n=g);  D as for m16n8k8.
constexpr int kWLD16 = 56;         // row stride (elements) of the 16-bit dense weight tile [8][kWLD16]
__device__ __forceinline__ void mma16(float (&d)[4], const unsigned (&a)[4], const unsigned (&b)[2], const __half*) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void mma16(float (&d)[4], const unsigned (&a)[4], const unsigned (&b)[2],
                                      const __nv_bfloat16*) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void mma16(float (&)[4], const unsigned (&)[4], const unsigned (&)[2], const float*) {}
__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// element offset of 8-element chunk c of staged 16-bit row r
__device__ __forceinline__ int swz16(int r, int c) { return r * kC + ((c ^ ((r >> 1) & 3)) << 3); }

// tiled_sum: D[ch][q] += sum_u X[u][ch] * Wd16[q][u], u < 16 ksteps.  A = X^T through ldmatrix.trans.
template <typename T>
__device__ __forceinline__ void sum_product16(const T* Xraw, const T* Wd16, int ksteps, int lane, float (&acc)[2][4]) {
    const int mi = lane >> 3, rr = lane & 7, g = lane >> 2, t = lane & 3;
    unsigned xa[2];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) xa[mt] = smem_u32(Xraw + swz16((mi >> 1) * 8 + rr, 2 * mt + (mi & 1)));
    const unsigned wa = smem_u32(Wd16 + g * kWLD16 + 2 * t);
#pragma unroll
    for (int ks = 0; ks < kUC / 16; ++ks) {
        if (ks < ksteps) {
            unsigned b[2];
            asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(b[0]) : "r"(wa + ks * 32));
            asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(b[1]) : "r"(wa + ks * 32 + 16));
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
                unsigned a[4];
                ldsm_x4_trans(a, xa[mt] + ks * 16 * kC * 2);
                mma16(acc[mt], a, b, static_cast<const T*>(nullptr));
            }
        }
    }
}

// tiled_dot: Sb[q][u] = sum_ch Y[q][ch] * X[u][ch] for u < 16 mtiles; yb = B fragments of the Y tile
// (yb[ks][h] = Y[g][16 ks + 8 h + 2t .. + 1], loaded by the caller), A = X through ldmatrix.
template <typename T>
__device__ __forceinline__ void dot_product16(const T* Xraw, const unsigned (&yb)[2][2], float* Sb, int mtiles, int lane) {
    const int mi = lane >> 3, rr = lane & 7, g = lane >> 2, t = lane & 3;
    unsigned xd[2];
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) xd[ks] = smem_u32(Xraw + swz16((mi & 1) * 8 + rr, 2 * ks + (mi >> 1)));
#pragma unroll
    for (int mt = 0; mt < kUC / 16; ++mt) {
        if (mt < mtiles) {
            float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
                unsigned a[4];
                ldsm_x4(a, xd[ks] + mt * 16 * kC * 2);
                mma16(d, a, yb[ks], static_cast<const T*>(nullptr));
            }
            // d0=(u=16mt+g, q=2t) d1=(u, 2t+1) d2=(u+8, 2t) d3=(u+8, 2t+1)
            float* sp = Sb + (2 * t) * kWLD + 16 * mt + g;
            sp[0] = d[0];
            sp[kWLD] = d[1];
            sp[8] = d[2];
            sp[kWLD + 8] = d[3];
        }
    }
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

// as_runs (optional): when the tile is made of aligned runs of 8 tokens, *as_runs is set and lut holds ONE slot
// per run edge y = row * (m / 8) + run (the run's 8 tokens have slots 8 s .. 8 s + 7) instead of one per edge.
__device__ int dedup_tile(const DedupScratch ps_, const long long* ring, unsigned short* lut, int E, int m, int i0,
                          int n, bool want_rowdup, bool* rowdup, int lane, int n_src = -1, bool* as_runs = nullptr) {
    if (n_src < 0) n_src = n;
    if (as_runs) *as_runs = false;
    const DedupScratch* ps = &ps_;
    int lo = INT_MAX, hi = -1;
    // Tiles whose rows are made of aligned runs of 8 consecutive tokens (neighbourhoods built from whole
    // clusters, as the model does): the runs are de-duplicated instead of the tokens, one eighth of the work.
    bool maybe_runs = (m & 7) == 0 && i0 + kT <= n;
    if (maybe_runs) {                                   // cheap look at the first 32 indices before the full check
        const long long v = ring[lane], v0 = ring[lane & ~7];
        maybe_runs = __all_sync(kFull, (v0 & 7) == 0 && v == v0 + (lane & 7));
    }
    if (maybe_runs) {
        bool runs = true;
        for (int x = lane; x < E; x += 32) {            // (x & 7) == (lane & 7)
            const long long v = ring[x], v0 = ring[x & ~7];
            runs = runs && v0 >= 0 && (v0 & 7) == 0 && v == v0 + (x & 7) && v0 + 7 < n_src;
        }
        if (__all_sync(kFull, runs)) {
            const int R = E >> 3;                       // run edges, m / 8 per row
            unsigned short* slot_r = ps->tok + 64;      // R <= 48
            for (int y = lane; y < R; y += 32) {
                const int rid = (int)(ring[8 * y] >> 3);
                ps->tok[y] = (unsigned short)rid;
                lo = min(lo, rid);
                hi = max(hi, rid);
            }
            const int UR = dedup_tokens(ps_, slot_r, R, m >> 3, want_rowdup, rowdup, lane, lo, hi);
            int rid[2];
#pragma unroll
            for (int k = 0; k < 2; ++k) rid[k] = lane + 32 * k < UR ? (int)ps->uniq[lane + 32 * k] : 0;
            __syncwarp();
#pragma unroll
            for (int k = 0; k < 2; ++k)
                if (lane + 32 * k < UR) {
#pragma unroll
                    for (int r = 0; r < 8; ++r) ps->uniq[(lane + 32 * k) * 8 + r] = (unsigned short)(rid[k] * 8 + r);
                }
            if (as_runs) {
                *as_runs = true;
                for (int y = lane; y < R; y += 32) lut[y] = slot_r[y];
            } else {
                for (int x = lane; x < E; x += 32) lut[x] = (unsigned short)(slot_r[x >> 3] * 8 + (x & 7));
            }
            __syncwarp();
            return UR * 8;
        }
    }
    for (int x = lane; x < E; x += 32) {
        const long long v = ring[x];
        const int q = x / m;
        unsigned short t = kSkip;
        if (i0 + q < n && v >= 0 && v < n_src) {
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
            ps->uniq[x] = t != kSkip ? t : (unsigned short)0;      // a slot nobody refers to: any valid row
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


}  // namespace
}  // namespace clusten
