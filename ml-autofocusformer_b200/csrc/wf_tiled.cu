// Tiled CLUSTENWF kernels (gather side): feat_new = weights^T x gathered features, and d_weights.
//
//   wf_sum   out[b,i,k,:] = sum_j W[b,i,j,k] * F[b, idx[b,i,j], :]          (forward)
//   wf_dot   dW[b,i,j,k]  = <F[b, idx[b,i,j], :], dO[b,i,k,:]>              (d_weights)
//
// The merge centres arrive in no particular order (models/aff_transformer.py:320-336 of the reference
// picks them with an unsorted top-k), so consecutive rows of nbhd_idx share nothing.  A small pre-pass
// orders the rows of each batch element by their first neighbour (wf_order_kernel, bitonic sort in
// shared memory); a warp then takes 8 rows that are adjacent in that order -- spatial neighbours -- and,
// as in the attention kernels, de-duplicates their 8 x m indices, stages every distinct feature row once
// per 32-channel slab and multiplies on the tensor cores.  The reference gathers every feature row ic
// times per output (clusten/src/clustenwf_cuda_kernel.cu:41-47).
#include "tile_core.cuh"

namespace clusten {
namespace {

constexpr int kMaxIC = 4;

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

// ----------------------------------------------------------------------------- shared pieces
struct WfParams {
    const void* W;        // [b, n_out, m, ic]   (wf_dot: output d_weights)
    const void* F;        // [b, n, c]
    const void* G;        // wf_dot: d_feat_new [b, n_out, ic, c]
    void* out;            // wf_sum: feat_new [b, n_out, ic, c];  wf_dot: d_weights
    const int64_t* idx;   // [b, n_out, m]
    const int* order;     // [b, n_out] or nullptr (identity)
    int batch, n_out, n, m, ic, c, tiles;
};

// per-warp shared memory:  X rows [48][32] fp32 (front: landed indices) | Xraw (16-bit inputs) |
//                          Op: dense weights [8 ic][kWLD] (wf_sum) or Y [8 ic][kYLD] + scores [8 ic][kWLD] (wf_dot)
//                          | lut | uniq
template <typename T, int MODE> struct WfSmem {
    static constexpr bool kIsFloat = std::is_same<T, float>::value;
    static constexpr int kX = kUC * kC * 4;
    static constexpr int kXraw = kIsFloat ? 0 : kUC * kC * (int)sizeof(T);
    static constexpr int kOp = MODE == 0 ? kT * kMaxIC * kWLD * 4 : kT * kMaxIC * (kYLD + kWLD) * 4;
    static constexpr int kLut = kE * 2;
    static constexpr int kTotal = kX + kXraw + kOp + 2 * kLut;
};

// three-pass product with operands that are already split
__device__ __forceinline__ void mma3(float (&d)[4], const unsigned (&ah)[4], const unsigned (&al)[4],
                                     const unsigned (&bh)[2], const unsigned (&bl)[2]) {
    mma_tf32(d, al, bh);
    mma_tf32(d, ah, bl);
    mma_tf32(d, ah, bh);
}

// ----------------------------------------------------------------------------- kernel
// MODE 0: wf_sum, MODE 1: wf_dot.  ICT = ic (1, 2 or 4).
template <typename T, int MODE, int ICT>
__global__ void __launch_bounds__(32 * kWarps, 3)
wf_tiles_kernel(const WfParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    using WS = WfSmem<T, MODE>;
    constexpr bool kIsFloat = WS::kIsFloat;
    constexpr int kPer = 16 / (int)sizeof(T);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int qi = lane >> 3, ci = lane & 7, g = lane >> 2, t = lane & 3;
    unsigned char* base = smem_raw + size_t(warp) * WS::kTotal;
    float* Xs = reinterpret_cast<float*>(base);
    T* Xraw = reinterpret_cast<T*>(base + WS::kX);
    float* Op = reinterpret_cast<float*>(base + WS::kX + WS::kXraw);
    unsigned short* lut = reinterpret_cast<unsigned short*>(base + WS::kX + WS::kXraw + WS::kOp);
    unsigned short* uniq = lut + kE;
    long long* ring = reinterpret_cast<long long*>(Xs);
    DedupScratch ds;
    ds.tok = reinterpret_cast<unsigned short*>(base + kE * 8);
    ds.uniq = uniq;
    ds.bm = reinterpret_cast<unsigned*>(Op);
    ds.pre = reinterpret_cast<unsigned short*>(ds.bm + kBMW);
    ds.rowbm = reinterpret_cast<unsigned*>(ds.pre + kBMW);
    float* Wd = Op;                                    // MODE 0: [ICT * 8][kWLD], row = k * 8 + q
    float* Ys = Op;                                    // MODE 1: [ICT * 8][kYLD]
    float* Sb = Op + kT * kMaxIC * kYLD;               // MODE 1: [ICT * 8][kWLD]

    const int m = p.m, c = p.c, n = p.n, n_out = p.n_out;
    const int E = kT * m;
    const T* Wg = static_cast<const T*>(p.W);
    const T* Fg = static_cast<const T*>(p.F);
    const T* Gg = static_cast<const T*>(p.G);
    T* Og = static_cast<T*>(p.out);
    const int sw_sum = (ci ^ (qi << 1)) << 2;          // MODE 0 swizzle of staged row qi + 4k
    const int sw_dot_e = (ci ^ qi) << 2, sw_dot_o = sw_dot_e ^ 16;
    const SumAddr sa = make_sum_addr(Wd, Xs, lane);
    const DotAddr da = make_dot_addr(Ys, Xs, Sb, lane);

    const unsigned total = (unsigned)p.batch * (unsigned)p.tiles;
    const unsigned nwarps = gridDim.x * kWarps;
    for (unsigned task = blockIdx.x * kWarps + warp; task < total; task += nwarps) {
        const int b = (int)(task / (unsigned)p.tiles);
        const int i0 = (int)(task - (unsigned)b * (unsigned)p.tiles) * kT;
        // rows of this tile (lane q < 8 holds row q; -1 past the end)
        int myrow = -1;
        if (lane < kT && i0 + lane < n_out)
            myrow = p.order ? p.order[(long long)b * n_out + i0 + lane] : i0 + lane;
        int rows[kT];
#pragma unroll
        for (int q = 0; q < kT; ++q) rows[q] = __shfl_sync(kFull, myrow, q);
        // ---- indices of the 8 rows -> ring [8][m]
        __syncwarp();
#pragma unroll
        for (int q = 0; q < kT; ++q) {
            if (rows[q] >= 0) {
                const int64_t* src = p.idx + ((long long)b * n_out + rows[q]) * m;
                for (int j = lane; j < m; j += 32) cp_async8_ca(ring + q * m + j, src + j);
            } else {
                for (int j = lane; j < m; j += 32) ring[q * m + j] = -1;
            }
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncwarp();
        bool rowdup = false;
        // every row of the ring is "valid" for dedup_tile (i0 = 0, 8 rows); missing rows hold -1
        const int U = dedup_tile(ds, ring, lut, E, m, 0, kT, MODE == 0, &rowdup, lane, n);
        __syncwarp();

        float acc[ICT][2][4];                           // MODE 0
        const int nslabs = c / kC;
        for (int s = 0; s < (MODE == 0 ? nslabs : 1); ++s) {
#pragma unroll
            for (int k = 0; k < ICT; ++k)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[k][0][i] = acc[k][1][i] = 0.f;
            const int nchunks = U > 0 ? (U + kUC - 1) / kUC : 1;
            for (int ch = 0; ch < nchunks; ++ch) {
                const int u0 = ch * kUC;
                const int Uc = max(0, min(kUC, U - u0));
                const int rows8 = (Uc + 7) & ~7;
                if (MODE == 0) {
                    // ---------------- forward: stage slab s of the rows, spread the weights, multiply
                    const T* Fb = Fg + (long long)b * n * c + s * kC;
                    __syncwarp();
                    if (kIsFloat) {
#pragma unroll
                        for (int k = 0; k < kUC / 4; ++k) {
                            const int r = qi + 4 * k;
                            if (r < rows8) {
                                float* dst = Xs + r * kC + sw_sum;
                                if (r < Uc) cp_async16_cg(dst, Fb + (long long)uniq[u0 + r] * c + ci * 4);
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
                                if (r < Uc) cp_async16_cg(dst, Fb + (long long)uniq[u0 + r] * c + pc * kPer);
                                else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
                            }
                        }
                    }
                    cp_async_commit();
                    for (int z = lane; z < ICT * kT * kWLD / 4; z += 32)
                        reinterpret_cast<float4*>(Wd)[z] = make_float4(0.f, 0.f, 0.f, 0.f);
                    __syncwarp();
                    if (!rowdup) {
                        int q = 0, j = lane;                    // edge x = lane + 32 step  ->  (q, j)
                        while (j >= m) { j -= m; ++q; }
                        for (int x = lane; x < E; x += 32) {
                            const unsigned short sl = lut[x];
                            const int rel = (int)sl - u0;
                            if (sl != kSkip && rel >= 0 && rel < Uc) {
                                int rq = rows[0];
#pragma unroll
                                for (int qq = 1; qq < kT; ++qq)
                                    if (q == qq) rq = rows[qq];
                                const T* w = Wg + (((long long)b * n_out + rq) * m + j) * ICT;
#pragma unroll
                                for (int k = 0; k < ICT; ++k) Wd[(k * kT + q) * kWLD + rel] = Elem<T>::up(w[k]);
                            }
                            j += 32;
                            while (j >= m) { j -= m; ++q; }
                        }
                    } else if (lane < kT) {
                        // some row repeats a neighbour: one lane per row adds the weights in column order
                        int rq = rows[0];
#pragma unroll
                        for (int qq = 1; qq < kT; ++qq)
                            if (lane == qq) rq = rows[qq];
                        if (rq >= 0) {
                            const T* w = Wg + (((long long)b * n_out + rq) * m) * ICT;
                            for (int j = 0; j < m; ++j) {
                                const unsigned short sl = lut[lane * m + j];
                                const int rel = (int)sl - u0;
                                if (sl != kSkip && rel >= 0 && rel < Uc) {
#pragma unroll
                                    for (int k = 0; k < ICT; ++k)
                                        Wd[(k * kT + lane) * kWLD + rel] += Elem<T>::up(w[j * ICT + k]);
                                }
                            }
                        }
                    }
                    cp_async_wait<0>();
                    __syncwarp();
                    if (!kIsFloat) {
#pragma unroll
                        for (int k = 0; k < kUC / 4; ++k) {
                            const int r = qi + 4 * k;
                            if (r < rows8) st4(Xs + r * kC + sw_sum, ld4(Xraw + r * kC + ci * 4));
                        }
                        __syncwarp();
                    }
                    // D_k[c][q] += sum_u X[u][c] * Wd[k*8+q][u]: A fragments loaded and split once per step
                    for (int us = 0; us < rows8; us += 8) {
                        float a[2][4];
                        unsigned ah[2][4], al[2][4];
#pragma unroll
                        for (int mt = 0; mt < 2; ++mt) {
                            asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(a[mt][0]) : "r"(sa.x[mt][0] + us * kC * 4));
                            asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(a[mt][1]) : "r"(sa.x[mt][1] + us * kC * 4));
                            asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(a[mt][2]) : "r"(sa.x[mt][0] + (us + 4) * kC * 4));
                            asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(a[mt][3]) : "r"(sa.x[mt][1] + (us + 4) * kC * 4));
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                if (kIsFloat) split_tf32(a[mt][i], ah[mt][i], al[mt][i]);
                                else { ah[mt][i] = __float_as_uint(a[mt][i]); al[mt][i] = 0u; }
                            }
                        }
#pragma unroll
                        for (int k = 0; k < ICT; ++k) {
                            float bv[2];
                            asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(bv[0]) : "r"(sa.w + (k * kT * kWLD + us) * 4));
                            asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(bv[1]) : "r"(sa.w + (k * kT * kWLD + us + 4) * 4));
                            unsigned bh[2], bl[2];
#pragma unroll
                            for (int i = 0; i < 2; ++i) {
                                if (kIsFloat) split_tf32(bv[i], bh[i], bl[i]);
                                else { bh[i] = __float_as_uint(bv[i]); bl[i] = 0u; }
                            }
#pragma unroll
                            for (int mt = 0; mt < 2; ++mt) {
                                if (kIsFloat) mma3(acc[k][mt], ah[mt], al[mt], bh, bl);
                                else mma_tf32(acc[k][mt], ah[mt], bh);
                            }
                        }
                    }
                }
            }
            if (MODE == 0) {
                // D fragments -> output tile [8][kOLD] per k -> 16-byte stores
                float* Ot = Op;
#pragma unroll
                for (int k = 0; k < ICT; ++k) {
                    __syncwarp();
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
                        float* o = Ot + (2 * t) * kOLD + 16 * mt + g;
                        o[0] = acc[k][mt][0];
                        o[kOLD] = acc[k][mt][1];
                        o[8] = acc[k][mt][2];
                        o[kOLD + 8] = acc[k][mt][3];
                    }
                    __syncwarp();
#pragma unroll
                    for (int a2 = 0; a2 < 2; ++a2) {
                        const int q = 2 * qi + a2;
                        int rq = rows[0];
#pragma unroll
                        for (int qq = 1; qq < kT; ++qq)
                            if (q == qq) rq = rows[qq];
                        if (rq >= 0)
                            st4(Og + (((long long)b * n_out + rq) * ICT + k) * c + s * kC + ci * 4,
                                *reinterpret_cast<const float4*>(Ot + q * kOLD + ci * 4));
                    }
                }
                __syncwarp();
            }
        }
        (void)Gg; (void)da; (void)sw_dot_e; (void)sw_dot_o; (void)Ys; (void)Sb;
    }
}

template <typename T, int ICT>
int wf_sum_t(const char* label, const WfParams& p, cudaStream_t s) {
    const size_t smem = size_t(kWarps) * WfSmem<T, 0>::kTotal;
    auto kernel = wf_tiles_kernel<T, 0, ICT>;
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

template <typename T>
int wf_sum_ic(const char* label, const WfParams& p, cudaStream_t s) {
    switch (p.ic) {
        case 1: return wf_sum_t<T, 1>(label, p, s);
        case 2: return wf_sum_t<T, 2>(label, p, s);
        case 4: return wf_sum_t<T, 4>(label, p, s);
        default: return CLUSTEN_ERR_UNSUPPORTED;
    }
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

bool tiled_wf_sum_supported(int dtype, const void* W, const void* F, const void* out, int n_out, int n, int m, int ic,
                            int c) {
    if (dtype != CLUSTEN_F32 && dtype != CLUSTEN_F16 && dtype != CLUSTEN_BF16) return false;
    if (c % kC != 0 || (ic != 1 && ic != 2 && ic != 4) || m < 1 || m > kMmax || n > 65000 || n_out < 1) return false;
    return reinterpret_cast<uintptr_t>(F) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0 &&
           reinterpret_cast<uintptr_t>(W) % 16 == 0;
}

int launch_tiled_wf_sum(const char* label, int dtype, const void* W, const void* F, const int64_t* idx,
                        const int* order, void* out, int b, int n_out, int n, int m, int ic, int c, cudaStream_t s) {
    WfParams p{};
    p.W = W;  p.F = F;  p.G = nullptr;  p.out = out;  p.idx = idx;  p.order = order;
    p.batch = b;  p.n_out = n_out;  p.n = n;  p.m = m;  p.ic = ic;  p.c = c;  p.tiles = (n_out + kT - 1) / kT;
    if ((long long)b * p.tiles > 0x7fffffffLL) return CLUSTEN_ERR_SHAPE;
    switch (dtype) {
        case CLUSTEN_F32: return wf_sum_ic<float>(label, p, s);
        case CLUSTEN_F16: return wf_sum_ic<__half>(label, p, s);
        case CLUSTEN_BF16: return wf_sum_ic<__nv_bfloat16>(label, p, s);
        default: return CLUSTEN_ERR_DTYPE;
    }
}

}  // namespace clusten
