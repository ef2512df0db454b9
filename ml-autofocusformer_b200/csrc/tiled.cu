// Tiled scatter-side kernel for head_dim 32 (d_key, d_value); the gather side is in tiled_fwd.cu.
//
// A CTA takes a tile of 8 consecutive rows (one cluster of AutoFocusFormer) of one
// batch element and all heads.  The neighbour indices of the tile are read once,
// de-duplicated in shared memory (a bitmap over token ids gives every distinct
// neighbour a slot, in ascending token order), and every head then stages each
// distinct neighbour row ONCE and serves the 8 rows of the tile from it with a
// register-tiled 8 x U x 32 product on the FP32 pipes:
//
//   tiled_sum      out[i,:]  = sum_j W[i,j] * X[idx[i,j],:]      AV forward, d_query
//   tiled_dot      out[i,j]  = <X[idx[i,j],:], Y[i,:]>           QK forward, d_attn
//   tiled_scatter  out[t,:]  = sum_{idx[i,j]==t} W[i,j] * X[i,:] d_key, d_value  (rows = targets,
//                                                                 edges from the inverse index)
//
// The reference (clusten/src/clustenqk_cuda_kernel.cu:18-49,91-132,
// clustenav_cuda_kernel.cu:18-50,93-160) gives every output element its own thread,
// re-gathers each neighbour row from L2 for every query and scatters gradients with
// atomicAdd.  Here the weights of a tile are spread into a dense [8 x U] matrix so that
// any index pattern (rows shared by a cluster, per-token runs, random with repeats)
// goes through the same product; when the 8 rows of a tile are identical the
// de-duplication is skipped (slot = column).  Summation order is fixed: slots ascend
// with the token id and repeated neighbours of a row are pre-summed in column order.
#include <limits.h>

#include "tiled.cuh"

namespace clusten {

namespace {

constexpr int kT = 8;          // rows per tile
constexpr int kC = 32;         // channels per head
constexpr int kUC = 64;        // distinct neighbour rows staged at a time
constexpr int kEC = 512;       // edges (row, neighbour) handled at a time
constexpr int kEPL = kEC / 32; // edges per lane
constexpr int kBMW = 512;      // bitmap words -> token ids of a tile may span 16384
constexpr int kWLD = 68;       // row stride of the dense weight / score tile (floats)
constexpr int kYLD = 36;       // row stride of the staged Y tile (floats)
constexpr int kMaxWarps = 4;
constexpr unsigned kFull = 0xffffffffu;
constexpr unsigned short kSkip = 0xffffu;

// ----------------------------------------------------------------------------- shared memory
struct Smem {
    int tok[kEC];                 // source row of each edge of the chunk, -1 = none
    int ent[kEC];                 // tiled_scatter: raw inverse-index entry
    int uniq[kEC];                // slot -> source row
    unsigned bm[kBMW];
    unsigned short pre[kBMW];
    unsigned short slot[kEC];     // edge -> slot (| kRowDup), kSkip = contributes nothing
    unsigned char erow[kEC];      // tiled_scatter: tile row of each edge
    int misc[32];                 // [0]=U [1]=tmin [2]=tmax [3]=shared rows [8..16]=segment offsets
    int warp_tot[kMaxWarps];
    // followed by per-warp: float X[kUC * kC]; float Wd[kT * kWLD]; float Y[kT * kYLD]
};
constexpr int kWarpFloats = kUC * kC + kT * kWLD + kT * kYLD;

size_t smem_bytes(int warps) {
    size_t per_warp = size_t(kWarpFloats) * sizeof(float);
    size_t w = per_warp * warps;
    const size_t own = size_t(kT) * kEC * sizeof(int);   // duplicate-detection cells alias the warp area
    if (w < own) w = own;
    return ((sizeof(Smem) + 15) & ~size_t(15)) + w;
}

__device__ __forceinline__ float* warp_area(Smem* sm, int warp) {
    char* base = reinterpret_cast<char*>(sm) + ((sizeof(Smem) + 15) & ~size_t(15));
    return reinterpret_cast<float*>(base) + size_t(warp) * kWarpFloats;
}

// ----------------------------------------------------------------------------- element access
template <typename T> __device__ __forceinline__ float ld1(const T* p) { return Elem<T>::up(*p); }

// 4 consecutive elements -> float4 (p 16-byte aligned for float, 8-byte for 16-bit types)
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

// ----------------------------------------------------------------------------- de-duplication
// tok[0..E) -> slot[0..E), uniq[0..U); returns U (also in misc[0]).  All threads of the CTA.
__device__ int dedup_edges(Smem* sm, int E) {
    const int tid = threadIdx.x, nth = blockDim.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        sm->misc[1] = INT_MAX;
        sm->misc[2] = -1;
    }
    __syncthreads();
    int lo = INT_MAX, hi = -1;
    for (int x = tid; x < E; x += nth) {
        const int t = sm->tok[x];
        if (t >= 0) {
            lo = min(lo, t);
            hi = max(hi, t);
        }
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
    if (hi < 0) {                                      // no valid edge at all
        for (int x = tid; x < E; x += nth) sm->slot[x] = kSkip;
        if (tid == 0) sm->misc[0] = 0;
        __syncthreads();
        return 0;
    }
    const int w0 = lo >> 5;
    const int words = (hi >> 5) - w0 + 1;
    if (words > kBMW) {                                // ids too spread out: every edge gets its own slot
        for (int x = tid; x < E; x += nth) {
            const int t = sm->tok[x];
            sm->slot[x] = t >= 0 ? (unsigned short)x : kSkip;
            sm->uniq[x] = t;
        }
        if (tid == 0) sm->misc[0] = E;
        __syncthreads();
        return E;
    }
    for (int w = tid; w < words; w += nth) sm->bm[w] = 0u;
    __syncthreads();
    for (int x = tid; x < E; x += nth) {
        const int t = sm->tok[x];
        if (t >= 0) atomicOr(&sm->bm[(t >> 5) - w0], 1u << (t & 31));
    }
    __syncthreads();
    {   // exclusive prefix of the word popcounts
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
        if (tid == nth - 1) sm->misc[0] = run;          // last thread ends with the total
    }
    __syncthreads();
    for (int x = tid; x < E; x += nth) {
        const int t = sm->tok[x];
        if (t >= 0) {
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

// Stage rows uniq[u0 .. u0+rows4) of X (one head, [n_src][32]) into Xs, 16-byte chunks XOR-swizzled
// by the row number; rows past U are zero-filled.  One warp.
template <typename T>
__device__ __forceinline__ void stage_rows(float* __restrict__ Xs, const T* __restrict__ Xh,
                                           const int* __restrict__ uniq, int u0, int U, int rows4, int lane) {
    const int chunk = lane & 7;
#pragma unroll 4
    for (int r = lane >> 3; r < rows4; r += 4) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (u0 + r < U) {
            const int t = uniq[u0 + r];
            if (t >= 0) v = ld4(Xh + (long long)t * kC + chunk * 4);
        }
        st4(Xs + r * kC + ((chunk ^ (r & 7)) << 2), v);
    }
}

// ----------------------------------------------------------------------------- products
// acc[a][:] += Wd[2qi+a][u] * Xs[u][4ci..4ci+3], u < rows4 (multiple of 4)
__device__ __forceinline__ void sum_product(const float* __restrict__ Wd, const float* __restrict__ Xs, int rows4,
                                            int qi, int ci, float4 (&acc)[2]) {
    const float* w0p = Wd + (2 * qi) * kWLD;
    const float* w1p = w0p + kWLD;
    for (int u = 0; u < rows4; u += 4) {
        const float4 w0 = *reinterpret_cast<const float4*>(w0p + u);
        const float4 w1 = *reinterpret_cast<const float4*>(w1p + u);
        const float wa[4] = {w0.x, w0.y, w0.z, w0.w};
        const float wb[4] = {w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int r = u + k;
            const float4 x = *reinterpret_cast<const float4*>(Xs + r * kC + ((ci ^ (r & 7)) << 2));
            acc[0].x += wa[k] * x.x; acc[0].y += wa[k] * x.y; acc[0].z += wa[k] * x.z; acc[0].w += wa[k] * x.w;
            acc[1].x += wb[k] * x.x; acc[1].y += wb[k] * x.y; acc[1].z += wb[k] * x.z; acc[1].w += wb[k] * x.w;
        }
    }
}

// ----------------------------------------------------------------------------- tiled_scatter
// out[bb, t, :] = sum over inverse-index entries (i, j) of target t:  W[bb, i, j] * X[bb, i, :]
template <typename T>
__global__ void __launch_bounds__(32 * kMaxWarps)
tiled_scatter_kernel(const T* __restrict__ W, const T* __restrict__ X, const int64_t* __restrict__ idx,
                     InverseView inv, T* __restrict__ out, int heads, int n, int m, int tiles,
                     int tiles_per_cta) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Smem* sm = reinterpret_cast<Smem*>(smem_raw);
    const int tid = threadIdx.x, nth = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, nwarps = nth >> 5;
    const int qi = lane >> 3, ci = lane & 7;
    float* Xs = warp_area(sm, warp);
    float* Wd = Xs + kUC * kC;

    const int groups = (tiles + tiles_per_cta - 1) / tiles_per_cta;
    const int b = blockIdx.x / groups;
    const int tile0 = (blockIdx.x - b * groups) * tiles_per_cta;
    const int64_t* idx_b = idx + (long long)b * n * m;
    const int* rowptr = inv.rowptr + (long long)b * (n + 1);
    const int* seglen = inv.seglen + (long long)b * n;
    const int* entries = inv.entries + (long long)b * n * m;

    for (int tile = tile0; tile < min(tile0 + tiles_per_cta, tiles); ++tile) {
        const int t0 = tile * kT;
        // segment offsets of the 8 targets inside the tile's concatenated edge list
        if (tid == 0) {
            int run = 0;
            for (int r = 0; r < kT; ++r) {
                sm->misc[8 + r] = run;
                if (t0 + r < n) run += seglen[t0 + r];
            }
            sm->misc[8 + kT] = run;
        }
        __syncthreads();
        const int E_total = sm->misc[8 + kT];
        for (int e0 = 0; e0 == 0 || e0 < E_total; e0 += kEC) {
            const int E = min(kEC, E_total - e0);
            const bool first = e0 == 0;
            for (int x = tid; x < E; x += nth) {
                const int p = e0 + x;
                int r = 0;
#pragma unroll
                for (int k = 1; k < kT; ++k) r += (p >= sm->misc[8 + k]) ? 1 : 0;
                const int e = entries[rowptr[t0 + r] + (p - sm->misc[8 + r])];
                sm->ent[x] = e;
                sm->erow[x] = (unsigned char)r;
                sm->tok[x] = (int)((unsigned)e & ~kDupFlag) / m;
            }
            __syncthreads();
            const int U = E > 0 ? dedup_edges(sm, E) : 0;
            for (int g = warp; g < heads; g += nwarps) {
                const long long bb = (long long)b * heads + g;
                const T* Wh = W + (bb * n) * m;
                const T* Xh = X + (bb * n) * kC;
                float wreg[kEPL];
#pragma unroll
                for (int k = 0; k < kEPL; ++k) {
                    const int x = lane + 32 * k;
                    float w = 0.f;
                    if (x < E) {
                        const unsigned e = (unsigned)sm->ent[x];
                        if (!(e & kDupFlag)) {
                            w = ld1(Wh + e);
                        } else {                       // the target occurs several times in that row
                            const int row = sm->tok[x];
                            const int t = t0 + sm->erow[x];
                            const int64_t* irow = idx_b + (long long)row * m;
                            for (int j = 0; j < m; ++j)
                                if (irow[j] == t) w += ld1(Wh + (long long)row * m + j);
                        }
                    }
                    wreg[k] = w;
                }
                float4 acc[2];
                acc[0] = acc[1] = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int u0 = 0; u0 < U; u0 += kUC) {
                    const int Uc = min(kUC, U - u0);
                    const int rows4 = (Uc + 3) & ~3;
                    __syncwarp();
                    stage_rows<T>(Xs, Xh, sm->uniq, u0, U, rows4, lane);
                    for (int z = lane; z < kT * kWLD / 4; z += 32)
                        reinterpret_cast<float4*>(Wd)[z] = make_float4(0.f, 0.f, 0.f, 0.f);
                    __syncwarp();
#pragma unroll
                    for (int k = 0; k < kEPL; ++k) {
                        const int x = lane + 32 * k;
                        if (x < E) {
                            const int sl = (int)sm->slot[x] - u0;
                            if (sl >= 0 && sl < Uc) Wd[sm->erow[x] * kWLD + sl] = wreg[k];
                        }
                    }
                    __syncwarp();
                    sum_product(Wd, Xs, rows4, qi, ci, acc);
                }
#pragma unroll
                for (int a = 0; a < 2; ++a) {
                    const int t = t0 + 2 * qi + a;
                    if (t < n) {
                        T* o = out + (bb * n + t) * kC + ci * 4;
                        float4 v = acc[a];
                        if (!first) {
                            const float4 old = ld4(o);
                            v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
                        }
                        st4(o, v);
                    }
                }
            }
            __syncthreads();
        }
    }
}

// ----------------------------------------------------------------------------- host side
bool common_supported(int dtype, std::initializer_list<const void*> ptrs, int n, int m, int c) {
    if (c != kC) return false;
    if (dtype != CLUSTEN_F32 && dtype != CLUSTEN_F16 && dtype != CLUSTEN_BF16) return false;
    if (n < 1 || m < 1) return false;
    for (const void* p : ptrs)
        if (reinterpret_cast<uintptr_t>(p) % 16 != 0) return false;
    return true;
}

struct LaunchShape {
    int warps, tiles, tiles_per_cta, grid;
    size_t smem;
};

LaunchShape launch_shape(int b, int h, int n) {
    LaunchShape s;
    s.warps = h < kMaxWarps ? h : kMaxWarps;
    s.tiles = (n + kT - 1) / kT;
    s.tiles_per_cta = 1;
    s.grid = b * ((s.tiles + s.tiles_per_cta - 1) / s.tiles_per_cta);
    s.smem = smem_bytes(s.warps);
    return s;
}

template <typename K>
int prepare(K kernel, size_t smem) {
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return CLUSTEN_ERR_CUDA;
        }
    }
    return CLUSTEN_OK;
}

template <typename T>
int tiled_scatter_t(const char* label, const void* W, const void* X, const int64_t* idx, const InverseView& inv,
                    void* out, int b, int h, int n, int m, cudaStream_t s) {
    const LaunchShape ls = launch_shape(b, h, n);
    int st = prepare(tiled_scatter_kernel<T>, ls.smem);
    if (st != CLUSTEN_OK) return st;
    ScopedKernelTimer timer(label, s);
    tiled_scatter_kernel<T><<<ls.grid, 32 * ls.warps, ls.smem, s>>>((const T*)W, (const T*)X, idx, inv, (T*)out,
                                                                   h, n, m, ls.tiles, ls.tiles_per_cta);
    note_launch();
    return check_launch();
}

}  // namespace

#define CLUSTEN_TILED_DISPATCH(dtype, FN, ...)                                    \
    switch (dtype) {                                                              \
        case CLUSTEN_F32: return FN<float>(__VA_ARGS__);                          \
        case CLUSTEN_F16: return FN<__half>(__VA_ARGS__);                         \
        case CLUSTEN_BF16: return FN<__nv_bfloat16>(__VA_ARGS__);                 \
        default: return CLUSTEN_ERR_DTYPE;                                        \
    }

bool tiled_scatter_supported(int dtype, const void* W, const void* X, const void* out, int n, int m, int c) {
    (void)W;
    return common_supported(dtype, {X, out}, n, m, c);
}
int launch_tiled_scatter(const char* label, int dtype, const void* W, const void* X, const int64_t* idx,
                         const InverseView& inv, void* out, int b, int h, int n, int m, cudaStream_t s) {
    CLUSTEN_TILED_DISPATCH(dtype, tiled_scatter_t, label, W, X, idx, inv, out, b, h, n, m, s)
}

}  // namespace clusten
