// k nearest neighbours of 2-D points: for every query the k database points of its batch element at
// the smallest Euclidean distance, ascending, ties towards the lower database index.
//
// This is the neighbourhood search AutoFocusFormer runs before every stage: each token looks for its
// nearest cluster centres (models/aff_transformer.py:476 of the reference, k = 6 of at most 1152
// centres) and, in the adaptive downsampling, for its nearest other token (:298, k = 2).  The reference
// evaluates it with a pykeops LazyTensor reduction (models/point_utils.py:27-58).  Here a thread owns a
// query and keeps its k best candidates in registers while the CTA streams the database through shared
// memory; distances are exact fp32 (sqrt(dx*dx + dy*dy)), no matrix-multiply shortcut.
#include <math_constants.h>

#include "common.cuh"

namespace clusten {
namespace {

constexpr int kKnnThreads = 256;
constexpr int kKnnTile = 2048;          // database points staged at a time (16 KB)

template <int K>
__global__ void __launch_bounds__(kKnnThreads)
knn2d_kernel(const float2* __restrict__ query, const float2* __restrict__ db, int nq, int n,
             int64_t* __restrict__ idx_out, float* __restrict__ dist_out) {
    __shared__ float2 pts[kKnnTile];
    const int b = blockIdx.y;
    const int qi = blockIdx.x * kKnnThreads + threadIdx.x;
    const bool live = qi < nq;
    const float2 q = live ? query[(long long)b * nq + qi] : make_float2(0.f, 0.f);
    const float2* dbb = db + (long long)b * n;
    float best[K];
    int who[K];
#pragma unroll
    for (int i = 0; i < K; ++i) {
        best[i] = CUDART_INF_F;
        who[i] = 0x7fffffff;
    }
    for (int t0 = 0; t0 < n; t0 += kKnnTile) {
        const int cnt = min(kKnnTile, n - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < cnt; i += kKnnThreads) pts[i] = dbb[t0 + i];
        __syncthreads();
        if (live) {
            for (int i = 0; i < cnt; ++i) {
                const float2 p = pts[i];
                const float dx = q.x - p.x, dy = q.y - p.y;
                const float d2 = dx * dx + dy * dy;
                if (d2 < best[K - 1]) {            // strict: among equals the earlier (lower) index stays
                    float d = d2;
                    int w = t0 + i;
                    bool moving = false;            // once inserted, everything behind moves down one place
#pragma unroll
                    for (int s = 0; s < K; ++s) {
                        if (moving || d < best[s]) {
                            moving = true;
                            const float td = best[s];
                            const int tw = who[s];
                            best[s] = d;
                            who[s] = w;
                            d = td;
                            w = tw;
                        }
                    }
                }
            }
        }
    }
    if (live) {
        const long long o = ((long long)b * nq + qi) * K;
#pragma unroll
        for (int i = 0; i < K; ++i) {
            idx_out[o + i] = who[i];
            if (dist_out) dist_out[o + i] = sqrtf(best[i]);
        }
    }
}

template <int K>
int knn2d_t(const float* query, const float* db, int b, int nq, int n, int64_t* idx_out, float* dist_out,
            cudaStream_t s) {
    const dim3 grid((nq + kKnnThreads - 1) / kKnnThreads, b);
    ScopedKernelTimer timer("knn2d", s);
    knn2d_kernel<K><<<grid, kKnnThreads, 0, s>>>(reinterpret_cast<const float2*>(query),
                                                 reinterpret_cast<const float2*>(db), nq, n, idx_out, dist_out);
    note_launch();
    return check_launch();
}

}  // namespace

int launch_knn2d(const float* query, const float* db, int b, int nq, int n, int k, int64_t* idx_out, float* dist_out,
                 cudaStream_t s) {
    switch (k) {
        case 1: return knn2d_t<1>(query, db, b, nq, n, idx_out, dist_out, s);
        case 2: return knn2d_t<2>(query, db, b, nq, n, idx_out, dist_out, s);
        case 3: return knn2d_t<3>(query, db, b, nq, n, idx_out, dist_out, s);
        case 4: return knn2d_t<4>(query, db, b, nq, n, idx_out, dist_out, s);
        case 5: return knn2d_t<5>(query, db, b, nq, n, idx_out, dist_out, s);
        case 6: return knn2d_t<6>(query, db, b, nq, n, idx_out, dist_out, s);
        case 7: return knn2d_t<7>(query, db, b, nq, n, idx_out, dist_out, s);
        case 8: return knn2d_t<8>(query, db, b, nq, n, idx_out, dist_out, s);
        default: return CLUSTEN_ERR_UNSUPPORTED;
    }
}

}  // namespace clusten
