// CLUSTENWF forward (and, further down, d_weights) as a plain walk over the neighbours.
//
//   feat_new[b, i, k, :] = sum_j weights[b, i, j, k] * feat[b, nbhd_idx[b, i, j], :]
//
// Half a warp takes one merge row and every lane 4 channels of a 64-channel group: the half fetches the next 16
// neighbours' indices and ic weights one per lane (contiguous, all in flight together) and hands them round by
// shuffles; per neighbour it reads the feature vector (16 bytes per lane in fp32, 256 contiguous bytes per
// row), four in flight at a time, and adds with fp32 FMAs in neighbour order -- the order of the reference's
// loop (clusten/src/clustenwf_cuda_kernel.cu:41-47), which gathers every feature row ic times per output
// element.  Rows are taken in the row order, so the two rows of a warp and the rows of neighbouring warps share
// most of their neighbours and find them in L1.  No shared memory and 64 registers: 32 warps per SM, against 12
// for the tiled kernel (wf_tiles_kernel), whose staging, de-duplication and three-pass TF32 products cost more
// instruction slots than these 16 FMAs per neighbour.  Measured faster for 16-bit inputs as well, although
// their products are single tensor-core instructions in the tiled kernel.
#include "tile_core.cuh"
#include "tiled.cuh"

namespace clusten {
namespace {

constexpr int kDirectWarps = 8;

struct WfDirectParams {
    const void* W;        // weights [b, n_out, m, ic]
    const void* F;        // feat [b, n, c]
    void* out;            // feat_new [b, n_out, ic, c]
    const int64_t* idx;   // [b, n_out, m]
    const int* order;     // [b, n_out] or nullptr
    int batch, n_out, n, m, c;
};

template <typename T, int ICT, bool C64>
__global__ void __launch_bounds__(32 * kDirectWarps, 4)
wf_forward_direct_kernel(const WfDirectParams p) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int half = lane >> 4, hl = lane & 15;
    const int m = p.m, c = C64 ? 64 : p.c, n = p.n, n_out = p.n_out;
    const unsigned pairs = (unsigned)(n_out + 1) >> 1;
    const unsigned total = (unsigned)p.batch * pairs;
    const unsigned nwarps = gridDim.x * kDirectWarps;
    for (unsigned task = blockIdx.x * kDirectWarps + warp; task < total; task += nwarps) {
        const int b = (int)(task / pairs);
        const int pos = (int)(task - (unsigned)b * pairs) * 2 + half;
        const long long brow = (long long)b * n_out;
        int rq = -1;
        if (pos < n_out) {
            rq = p.order ? p.order[brow + pos] : pos;
            if ((unsigned)rq >= (unsigned)n_out) rq = -1;        // an entry that is no row number: treated as absent
        }
        const int64_t* irow = p.idx + (brow + max(rq, 0)) * m;
        const T* wrow = static_cast<const T*>(p.W) + (brow + max(rq, 0)) * m * ICT;
        const T* Fb = static_cast<const T*>(p.F) + (long long)b * n * c + 4 * hl;
        for (int c0 = 0; c0 < c; c0 += 64) {
            float4 acc[ICT];
#pragma unroll
            for (int k = 0; k < ICT; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int j0 = 0; j0 < m; j0 += 16) {
                // the half's next 16 neighbours, one per lane
                long long my_t = -1;
                if (rq >= 0 && j0 + hl < m) my_t = irow[j0 + hl];
                const int mine = (my_t >= 0 && my_t < n) ? (int)my_t : -1;
                const int cnt = min(16, m - j0);
                // ... and their weights, one neighbour per lane: the row's 16 m bytes are contiguous
                float my_w[ICT];
#pragma unroll
                for (int k = 0; k < ICT; ++k) my_w[k] = 0.f;
                if (rq >= 0 && j0 + hl < m) {
                    if constexpr (ICT == 4) {
                        const float4 v = ld4(wrow + (j0 + hl) * 4);
                        my_w[0] = v.x;  my_w[1] = v.y;  my_w[2] = v.z;  my_w[3] = v.w;
                    } else {
#pragma unroll
                        for (int k = 0; k < ICT; ++k) my_w[k] = Elem<T>::up(wrow[(j0 + hl) * ICT + k]);
                    }
                }
                // four feature vectors in flight at a time (L1 / L2), summed in neighbour order.  A full chunk of
                // valid neighbours -- the rule -- runs without a test per neighbour.
                const bool clean = cnt == 16 && __all_sync(kFull, mine >= 0);
                if (clean) {
#pragma unroll
                    for (int jj = 0; jj < 16; jj += 4) {
                        float4 f[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int t = __shfl_sync(kFull, mine, jj + u, 16);
                            f[u] = ld4(Fb + (unsigned)t * (unsigned)c + c0);
                        }
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
#pragma unroll
                            for (int k = 0; k < ICT; ++k) {
                                const float w = __shfl_sync(kFull, my_w[k], jj + u, 16);
                                acc[k].x += w * f[u].x;
                                acc[k].y += w * f[u].y;
                                acc[k].z += w * f[u].z;
                                acc[k].w += w * f[u].w;
                            }
                        }
                    }
                    continue;
                }
                for (int jj = 0; jj < cnt; jj += 4) {
                    float4 f[4];
                    bool ok[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int t = __shfl_sync(kFull, mine, jj + u, 16);
                        ok[u] = jj + u < cnt && t >= 0;
                        if (ok[u]) f[u] = ld4(Fb + (unsigned)t * (unsigned)c + c0);
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        float w[ICT];
#pragma unroll
                        for (int k = 0; k < ICT; ++k) w[k] = __shfl_sync(kFull, my_w[k], jj + u, 16);
                        if (ok[u]) {
#pragma unroll
                            for (int k = 0; k < ICT; ++k) {
                                acc[k].x += w[k] * f[u].x;
                                acc[k].y += w[k] * f[u].y;
                                acc[k].z += w[k] * f[u].z;
                                acc[k].w += w[k] * f[u].w;
                            }
                        }
                    }
                }
            }
            if (rq >= 0) {
#pragma unroll
                for (int k = 0; k < ICT; ++k)
                    st4(static_cast<T*>(p.out) + ((brow + rq) * ICT + k) * c + c0 + 4 * hl, acc[k]);
            }
        }
    }
}

// d_weights the same way:  d_weights[b, i, j, k] = <feat[b, nbhd_idx[b, i, j], :], d_feat_new[b, i, k, :]>.
// Half a warp per merge row, 4 channels per lane: the row's ic gradient vectors stay in registers, four
// neighbours' feature vectors are in flight at a time, every lane forms its 4-channel share of the 4 x ic dot
// products, and a butterfly over the 16 lanes (each step halves the values a lane keeps) leaves lane l with
// the complete product number l -- neighbour l / ic of the four, weight l % ic -- so that the 16 results of the
// four neighbours are one contiguous 64-byte store (ic = 4).
struct WfDwDirectParams {
    const float* F;       // feat [b, n, c]
    const float* G;       // d_feat_new [b, n_out, ic, c]
    float* out;           // d_weights [b, n_out, m, ic]
    const int64_t* idx;   // [b, n_out, m]
    const int* order;     // [b, n_out] or nullptr
    int batch, n_out, n, m, c;
};

template <bool C64>
__global__ void __launch_bounds__(32 * kDirectWarps, 4)
wf_dweights_direct_kernel(const WfDwDirectParams p) {
    constexpr int ICT = 4;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int half = lane >> 4, hl = lane & 15;
    const int m = p.m, c = C64 ? 64 : p.c, n = p.n, n_out = p.n_out;
    const unsigned pairs = (unsigned)(n_out + 1) >> 1;
    const unsigned total = (unsigned)p.batch * pairs;
    const unsigned nwarps = gridDim.x * kDirectWarps;
    for (unsigned task = blockIdx.x * kDirectWarps + warp; task < total; task += nwarps) {
        const int b = (int)(task / pairs);
        const int pos = (int)(task - (unsigned)b * pairs) * 2 + half;
        const long long brow = (long long)b * n_out;
        int rq = -1;
        if (pos < n_out) {
            rq = p.order ? p.order[brow + pos] : pos;
            if ((unsigned)rq >= (unsigned)n_out) rq = -1;
        }
        const int64_t* irow = p.idx + (brow + max(rq, 0)) * m;
        const float* grow = p.G + (brow + max(rq, 0)) * ICT * c + 4 * hl;
        const float* Fb = p.F + (long long)b * n * c + 4 * hl;
        float* orow = p.out + (brow + max(rq, 0)) * m * ICT;
        float4 g[ICT];
        if (C64) {
#pragma unroll
            for (int k = 0; k < ICT; ++k) g[k] = *reinterpret_cast<const float4*>(grow + k * c);
        }
        for (int j0 = 0; j0 < m; j0 += 16) {
            long long my_t = -1;
            if (rq >= 0 && j0 + hl < m) my_t = irow[j0 + hl];
            const int mine = (my_t >= 0 && my_t < n) ? (int)my_t : -1;
            const int cnt = min(16, m - j0);
            // four neighbours: shares of the 4 x ic products, butterfly, one store.  CHECK: some neighbour of the
            // chunk may be absent or out of range
            auto four = [&](int jj, auto check) {
                constexpr bool CHECK = decltype(check)::value;
                float v[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] = 0.f;
                int t[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) t[u] = __shfl_sync(kFull, mine, (jj + u) & 15, 16);
                for (int c0 = 0; c0 < c; c0 += 64) {
                    if (!C64) {
#pragma unroll
                        for (int k = 0; k < ICT; ++k) g[k] = *reinterpret_cast<const float4*>(grow + k * c + c0);
                    }
                    float4 f[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        if (CHECK) {
                            f[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                            if (t[u] >= 0) f[u] = *reinterpret_cast<const float4*>(Fb + (unsigned)t[u] * (unsigned)c + c0);
                        } else {
                            f[u] = *reinterpret_cast<const float4*>(Fb + (unsigned)t[u] * (unsigned)c + c0);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u)
#pragma unroll
                        for (int k = 0; k < ICT; ++k)
                            v[u * 4 + k] += f[u].x * g[k].x + f[u].y * g[k].y + f[u].z * g[k].z + f[u].w * g[k].w;
                }
                // butterfly: after the step with mask s a lane keeps the half of its values that its bit s selects
#pragma unroll
                for (int s = 8, cntv = 16; s > 0; s >>= 1, cntv >>= 1) {
                    const bool upper = (hl & s) != 0;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        if (i < cntv / 2) {
                            const float lo = v[i], hi = v[i + cntv / 2];
                            const float send = upper ? lo : hi, keep = upper ? hi : lo;
                            v[i] = keep + __shfl_xor_sync(kFull, send, s, 16);
                        }
                    }
                }
                // lane l holds product l: neighbour jj + l / 4, weight l % 4
                if (CHECK) {
                    if (rq >= 0 && jj + (hl >> 2) < cnt) orow[(j0 + jj) * ICT + hl] = v[0];
                } else {
                    orow[(j0 + jj) * ICT + hl] = v[0];
                }
            };
            const bool clean = cnt == 16 && __all_sync(kFull, mine >= 0);      // both rows present, all neighbours valid
            if (clean) {
#pragma unroll
                for (int jj = 0; jj < 16; jj += 4) four(jj, std::false_type{});
            } else {
                for (int jj = 0; jj < cnt; jj += 4) four(jj, std::true_type{});
            }
        }
    }
}

int wf_dweights_direct(const char* label, const WfDwDirectParams& p, cudaStream_t s) {
    auto kernel = p.c == 64 ? wf_dweights_direct_kernel<true> : wf_dweights_direct_kernel<false>;
    const int per_sm = resident_ctas(reinterpret_cast<const void*>(kernel), 32 * kDirectWarps, 0);
    if (per_sm < 0) return per_sm;
    const long long tasks = (long long)p.batch * ((p.n_out + 1) / 2);
    long long grid = (long long)sm_count() * per_sm;
    const long long need = (tasks + kDirectWarps - 1) / kDirectWarps;
    if (grid > need) grid = need;
    ScopedKernelTimer timer(label, s);
    kernel<<<(int)grid, 32 * kDirectWarps, 0, s>>>(p);
    note_launch();
    return check_launch();
}

template <typename T, int ICT>
int wf_forward_direct_t(const char* label, const WfDirectParams& p, cudaStream_t s) {
    auto kernel = p.c == 64 ? wf_forward_direct_kernel<T, ICT, true> : wf_forward_direct_kernel<T, ICT, false>;
    const int per_sm = resident_ctas(reinterpret_cast<const void*>(kernel), 32 * kDirectWarps, 0);
    if (per_sm < 0) return per_sm;
    const long long tasks = (long long)p.batch * ((p.n_out + 1) / 2);
    long long grid = (long long)sm_count() * per_sm;
    const long long need = (tasks + kDirectWarps - 1) / kDirectWarps;
    if (grid > need) grid = need;
    ScopedKernelTimer timer(label, s);
    kernel<<<(int)grid, 32 * kDirectWarps, 0, s>>>(p);
    note_launch();
    return check_launch();
}

}  // namespace

bool wf_forward_direct_supported(int dtype, int n_out, int n, int m, int ic, int c) {
    // element offsets inside a batch element are kept in 32 bits
    return (dtype == CLUSTEN_F32 || dtype == CLUSTEN_F16 || dtype == CLUSTEN_BF16) && (ic == 1 || ic == 2 || ic == 4) &&
           c % 64 == 0 &&
           (long long)n * c <= 0xffffffffLL && (long long)n_out * m * ic <= 0x7fffffffLL;
}

template <typename T>
static int wf_forward_direct_ic(const char* label, int ic, const WfDirectParams& p, cudaStream_t s) {
    switch (ic) {
        case 1: return wf_forward_direct_t<T, 1>(label, p, s);
        case 2: return wf_forward_direct_t<T, 2>(label, p, s);
        case 4: return wf_forward_direct_t<T, 4>(label, p, s);
        default: return CLUSTEN_ERR_UNSUPPORTED;
    }
}

int launch_wf_forward_direct(const char* label, int dtype, const void* W, const void* F, const int64_t* idx,
                             const int* order, void* out, int b, int n_out, int n, int m, int ic, int c,
                             cudaStream_t s) {
    WfDirectParams p{};
    p.W = W;  p.F = F;  p.out = out;  p.idx = idx;  p.order = order;
    p.batch = b;  p.n_out = n_out;  p.n = n;  p.m = m;  p.c = c;
    if ((long long)b * ((n_out + 1) / 2) > 0x7fffffffLL) return CLUSTEN_ERR_SHAPE;
    switch (dtype) {
        case CLUSTEN_F32: return wf_forward_direct_ic<float>(label, ic, p, s);
        case CLUSTEN_F16: return wf_forward_direct_ic<__half>(label, ic, p, s);
        case CLUSTEN_BF16: return wf_forward_direct_ic<__nv_bfloat16>(label, ic, p, s);
        default: return CLUSTEN_ERR_DTYPE;
    }
}

int launch_wf_dweights_direct(const char* label, const void* F, const void* G, const int64_t* idx, const int* order,
                              void* d_weights, int b, int n_out, int n, int m, int c, cudaStream_t s) {
    WfDwDirectParams p{};
    p.F = static_cast<const float*>(F);  p.G = static_cast<const float*>(G);  p.out = static_cast<float*>(d_weights);
    p.idx = idx;  p.order = order;
    p.batch = b;  p.n_out = n_out;  p.n = n;  p.m = m;  p.c = c;
    if ((long long)b * ((n_out + 1) / 2) > 0x7fffffffLL) return CLUSTEN_ERR_SHAPE;
    return wf_dweights_direct(label, p, s);
}

}  // namespace clusten
