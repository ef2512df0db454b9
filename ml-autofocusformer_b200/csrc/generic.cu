// Shape-agnostic CLUSTEN kernels: one warp per output row, any m / c / ic and
// all four element types.  They are the path for shapes the tiled kernels do
// not cover and the straightforward statement of the three access patterns:
//
//   gather_sum   out[row]      = sum_j  w[row, j] * x[idx[row, j]]     (AV forward, d_query, WF forward)
//   gather_dot   out[row, j]   = <x[idx[row, j]], y[row]>              (QK forward, d_attn, d_weights)
//   scatter_sum  out[t]        = sum over the inverse index of t        (d_key, d_value, d_feat)
//
// Compare clusten/src/clusten{qk,av,wf}_cuda_kernel.cu of the reference, which
// assigns one thread per output element and scatters with atomics.
#include "common.cuh"

namespace clusten {

namespace {

constexpr unsigned kFull = 0xffffffffu;
constexpr int kThreads = 256;

template <typename A>
__device__ __forceinline__ A warp_sum(A x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(kFull, x, o);
    return x;
}

template <typename T, int V, int ICT>
__global__ void __launch_bounds__(kThreads)
gather_sum_kernel(const T* __restrict__ W, const T* __restrict__ X, const int64_t* __restrict__ idx,
                  T* __restrict__ out, int nb, int heads, int n_rows, int n_src, int m, int ic_n, int ic0,
                  int c) {
    using A = typename Elem<T>::acc_t;
    const int lane = threadIdx.x & 31;
    const long long warp0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = (gridDim.x * (long long)blockDim.x) >> 5;
    const long long total = (long long)nb * n_rows;
    for (long long wr = warp0; wr < total; wr += nwarps) {
        const int bb = (int)(wr / n_rows);
        const int row = (int)(wr - (long long)bb * n_rows);
        const int bi = bb / heads;
        const int64_t* irow = idx + ((long long)bi * n_rows + row) * m;
        const T* wrow = W + (((long long)bb * n_rows + row) * m) * ic_n + ic0;
        const T* xb = X + (long long)bb * n_src * c;
        T* orow = out + (((long long)bb * n_rows + row) * ic_n + ic0) * c;
        for (int cb = 0; cb < c; cb += 32 * V) {
            const int ch = cb + lane * V;
            const bool act = ch < c;
            A acc[ICT][V];
#pragma unroll
            for (int i = 0; i < ICT; ++i)
#pragma unroll
                for (int v = 0; v < V; ++v) acc[i][v] = A(0);
            for (int j0 = 0; j0 < m; j0 += 32) {
                const int jl = j0 + lane;
                int tok = -1;
                A wl[ICT];
#pragma unroll
                for (int i = 0; i < ICT; ++i) wl[i] = A(0);
                if (jl < m) {
                    const long long tk = irow[jl];
                    if (tk >= 0 && tk < n_src) tok = (int)tk;
#pragma unroll
                    for (int i = 0; i < ICT; ++i) wl[i] = Elem<T>::up(wrow[(long long)jl * ic_n + i]);
                }
                const int cnt = min(32, m - j0);
                for (int jj = 0; jj < cnt; jj += 4) {       // four independent row loads per step
                    int t[4];
                    A wv[4][ICT];
                    Vec<T, V> x[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int src = (jj + u) & 31;
                        t[u] = __shfl_sync(kFull, tok, src);
                        if (jj + u >= cnt) t[u] = -1;
#pragma unroll
                        for (int i = 0; i < ICT; ++i) wv[u][i] = __shfl_sync(kFull, wl[i], src);
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (t[u] >= 0 && act) x[u] = ldg_vec<T, V>(xb + (long long)t[u] * c + ch);
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (t[u] >= 0 && act) {
#pragma unroll
                            for (int i = 0; i < ICT; ++i)
#pragma unroll
                                for (int v = 0; v < V; ++v) acc[i][v] += wv[u][i] * Elem<T>::up(x[u].v[v]);
                        }
                }
            }
            if (act) {
#pragma unroll
                for (int i = 0; i < ICT; ++i) {
                    Vec<T, V> o;
#pragma unroll
                    for (int v = 0; v < V; ++v) o.v[v] = Elem<T>::down(acc[i][v]);
                    st_vec<T, V>(orow + (long long)i * c + ch, o);
                }
            }
        }
    }
}

// One lane per neighbour: the lane walks its own gathered row (contiguous, V elements per load) against the
// row's Y vectors, which every lane reads from the same address (one broadcast transaction).
template <typename T, int V, int ICT>
__global__ void __launch_bounds__(kThreads)
gather_dot_kernel(const T* __restrict__ X, const T* __restrict__ Y, const int64_t* __restrict__ idx,
                  T* __restrict__ out, int nb, int heads, int n_rows, int n_src, int m, int ic_n, int ic0,
                  int c) {
    using A = typename Elem<T>::acc_t;
    const int lane = threadIdx.x & 31;
    const long long warp0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = (gridDim.x * (long long)blockDim.x) >> 5;
    const long long total = (long long)nb * n_rows;
    for (long long wr = warp0; wr < total; wr += nwarps) {
        const int bb = (int)(wr / n_rows);
        const int row = (int)(wr - (long long)bb * n_rows);
        const int bi = bb / heads;
        const int64_t* irow = idx + ((long long)bi * n_rows + row) * m;
        const T* xb = X + (long long)bb * n_src * c;
        const T* yrow = Y + (((long long)bb * n_rows + row) * ic_n + ic0) * c;
        T* orow = out + (((long long)bb * n_rows + row) * m) * ic_n + ic0;
        for (int j0 = 0; j0 < m; j0 += 32) {
            const int jl = j0 + lane;
            long long tk = -1;
            if (jl < m) tk = irow[jl];
            const bool ok = tk >= 0 && tk < n_src;
            const T* xrow = xb + (ok ? tk : 0) * c;
            A acc[ICT];
#pragma unroll
            for (int i = 0; i < ICT; ++i) acc[i] = A(0);
#pragma unroll 4
            for (int cb = 0; cb < c; cb += V) {
                const Vec<T, V> x = ldg_vec<T, V>(xrow + cb);
#pragma unroll
                for (int i = 0; i < ICT; ++i) {
                    const Vec<T, V> y = ldg_vec<T, V>(yrow + (long long)i * c + cb);
#pragma unroll
                    for (int v = 0; v < V; ++v) acc[i] += Elem<T>::up(x.v[v]) * Elem<T>::up(y.v[v]);
                }
            }
            if (jl < m) {
#pragma unroll
                for (int i = 0; i < ICT; ++i)
                    orow[(long long)jl * ic_n + i] = Elem<T>::down(ok ? acc[i] : A(0));
            }
        }
    }
}

template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
scatter_sum_kernel(const T* __restrict__ W, const T* __restrict__ X, const int64_t* __restrict__ idx,
                   InverseView inv, T* __restrict__ out, int nb, int heads, int n_rows, int n_tgt, int m,
                   int ic_n, int c) {
    using A = typename Elem<T>::acc_t;
    const int lane = threadIdx.x & 31;
    const long long warp0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = (gridDim.x * (long long)blockDim.x) >> 5;
    const long long total = (long long)nb * n_tgt;
    for (long long wr = warp0; wr < total; wr += nwarps) {
        const int bb = (int)(wr / n_tgt);
        const int t = (int)(wr - (long long)bb * n_tgt);
        const int bi = bb / heads;
        const int start = inv.rowptr[(long long)bi * (n_tgt + 1) + t];
        const int len = inv.seglen[(long long)bi * n_tgt + t];
        const int* ent = inv.entries + (long long)bi * n_rows * m + start;
        const T* wb = W + (long long)bb * n_rows * m * ic_n;
        const T* xb = X + (long long)bb * n_rows * ic_n * c;
        T* orow = out + ((long long)bb * n_tgt + t) * c;
        for (int cb = 0; cb < c; cb += 32 * V) {
            const int ch = cb + lane * V;
            const bool act = ch < c;
            A acc[V];
#pragma unroll
            for (int v = 0; v < V; ++v) acc[v] = A(0);
            for (int p0 = 0; p0 < len; p0 += 32) {
                const unsigned en = (p0 + lane < len) ? (unsigned)ent[p0 + lane] : 0u;
                const int cnt = min(32, len - p0);
                for (int jj = 0; jj < cnt; jj += 4) {       // four entries per step: independent loads
                    unsigned e[4];
                    bool plain = true;
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        e[u] = __shfl_sync(kFull, en, (jj + u) & 31);
                        if (jj + u < cnt && (e[u] & kDupFlag)) plain = false;
                    }
                    if (plain) {
                        int row[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) row[u] = (int)e[u] / m;
                        for (int i = 0; i < ic_n; ++i) {
                            A w[4];
                            Vec<T, V> x[4];
#pragma unroll
                            for (int u = 0; u < 4; ++u)
                                if (jj + u < cnt) {
                                    w[u] = Elem<T>::up(wb[(long long)e[u] * ic_n + i]);
                                    if (act) x[u] = ldg_vec<T, V>(xb + ((long long)row[u] * ic_n + i) * c + ch);
                                }
#pragma unroll
                            for (int u = 0; u < 4; ++u)
                                if (jj + u < cnt && act) {
#pragma unroll
                                    for (int v = 0; v < V; ++v) acc[v] += w[u] * Elem<T>::up(x[u].v[v]);
                                }
                        }
                        continue;
                    }
                    for (int u = 0; u < 4 && jj + u < cnt; ++u) {
                        if (!(e[u] & kDupFlag)) {
                            const int row = (int)e[u] / m;
                            for (int i = 0; i < ic_n; ++i) {
                                const A w = Elem<T>::up(wb[(long long)e[u] * ic_n + i]);
                                if (act) {
                                    const Vec<T, V> x = ldg_vec<T, V>(xb + ((long long)row * ic_n + i) * c + ch);
#pragma unroll
                                    for (int v = 0; v < V; ++v) acc[v] += w * Elem<T>::up(x.v[v]);
                                }
                            }
                        } else {
                            // the target occurs more than once in this row: take its slots in order
                            const int row = (int)(e[u] & ~kDupFlag) / m;
                            const int64_t* irow = idx + ((long long)bi * n_rows + row) * m;
                            for (int j = 0; j < m; ++j) {
                                if (irow[j] != t) continue;
                                const long long e2 = (long long)row * m + j;
                                for (int i = 0; i < ic_n; ++i) {
                                    const A w = Elem<T>::up(wb[e2 * ic_n + i]);
                                    if (act) {
                                        const Vec<T, V> x =
                                            ldg_vec<T, V>(xb + ((long long)row * ic_n + i) * c + ch);
#pragma unroll
                                        for (int v = 0; v < V; ++v) acc[v] += w * Elem<T>::up(x.v[v]);
                                    }
                                }
                            }
                        }
                    }
                }
            }
            if (act) {
                Vec<T, V> o;
#pragma unroll
                for (int v = 0; v < V; ++v) o.v[v] = Elem<T>::down(acc[v]);
                st_vec<T, V>(orow + ch, o);
            }
        }
    }
}

// widest vector (in elements) that divides c, keeps >= 32 lanes busy where c allows,
// and for which every row start stays aligned
int pick_vec(int c, int esize, std::initializer_list<const void*> ptrs) {
    int v = 1;
    if (c % 4 == 0 && c >= 128) v = 4;
    else if (c % 2 == 0 && c >= 64) v = 2;
    while (v > 1) {
        bool ok = true;
        for (const void* p : ptrs)
            if (reinterpret_cast<uintptr_t>(p) % (size_t(v) * esize) != 0) ok = false;
        if (ok) break;
        v >>= 1;
    }
    return v;
}

int grid_for(long long rows) {
    const long long warps_per_block = kThreads / 32;
    long long blocks = (rows + warps_per_block - 1) / warps_per_block;
    const long long cap = (long long)sm_count() * 32;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

template <typename T>
int gather_sum_t(const char* label, const void* W, const void* X, const int64_t* idx, void* out, int nb, int heads, int n_rows,
                 int n_src, int m, int ic, int c, cudaStream_t s) {
    const int v = pick_vec(c, sizeof(T), {X, out});
    const int grid = grid_for((long long)nb * n_rows);
    const int step = (ic % 4 == 0) ? 4 : 1;
    for (int ic0 = 0; ic0 < ic; ic0 += step) {
        ScopedKernelTimer timer(label, s);
#define CLUSTEN_GS(VV, II)                                                                              \
    gather_sum_kernel<T, VV, II><<<grid, kThreads, 0, s>>>((const T*)W, (const T*)X, idx, (T*)out, nb, \
                                                           heads, n_rows, n_src, m, ic, ic0, c)
        if (step == 4) {
            if (v == 4) CLUSTEN_GS(4, 4); else if (v == 2) CLUSTEN_GS(2, 4); else CLUSTEN_GS(1, 4);
        } else {
            if (v == 4) CLUSTEN_GS(4, 1); else if (v == 2) CLUSTEN_GS(2, 1); else CLUSTEN_GS(1, 1);
        }
#undef CLUSTEN_GS
        note_launch();
        const int st = check_launch();
        if (st != CLUSTEN_OK) return st;
    }
    return CLUSTEN_OK;
}

template <typename T>
int gather_dot_t(const char* label, const void* X, const void* Y, const int64_t* idx, void* out, int nb, int heads, int n_rows,
                 int n_src, int m, int ic, int c, cudaStream_t s) {
    int v = (c % 4 == 0) ? 4 : (c % 2 == 0 ? 2 : 1);
    while (v > 1 && (reinterpret_cast<uintptr_t>(X) % (v * sizeof(T)) != 0 ||
                     reinterpret_cast<uintptr_t>(Y) % (v * sizeof(T)) != 0))
        v >>= 1;
    const int grid = grid_for((long long)nb * n_rows);
    const int step = (ic % 4 == 0) ? 4 : 1;
    for (int ic0 = 0; ic0 < ic; ic0 += step) {
        ScopedKernelTimer timer(label, s);
#define CLUSTEN_GD(VV, II)                                                                              \
    gather_dot_kernel<T, VV, II><<<grid, kThreads, 0, s>>>((const T*)X, (const T*)Y, idx, (T*)out, nb, \
                                                           heads, n_rows, n_src, m, ic, ic0, c)
        if (step == 4) {
            if (v == 4) CLUSTEN_GD(4, 4); else if (v == 2) CLUSTEN_GD(2, 4); else CLUSTEN_GD(1, 4);
        } else {
            if (v == 4) CLUSTEN_GD(4, 1); else if (v == 2) CLUSTEN_GD(2, 1); else CLUSTEN_GD(1, 1);
        }
#undef CLUSTEN_GD
        note_launch();
        const int st = check_launch();
        if (st != CLUSTEN_OK) return st;
    }
    return CLUSTEN_OK;
}

template <typename T>
int scatter_sum_t(const char* label, const void* W, const void* X, const int64_t* idx, const InverseView& inv, void* out, int nb,
                  int heads, int n_rows, int n_tgt, int m, int ic, int c, cudaStream_t s) {
    const int v = pick_vec(c, sizeof(T), {X, out});
    const int grid = grid_for((long long)nb * n_tgt);
    ScopedKernelTimer timer(label, s);
#define CLUSTEN_SS(VV)                                                                                  \
    scatter_sum_kernel<T, VV><<<grid, kThreads, 0, s>>>((const T*)W, (const T*)X, idx, inv, (T*)out, nb, \
                                                        heads, n_rows, n_tgt, m, ic, c)
    if (v == 4) CLUSTEN_SS(4); else if (v == 2) CLUSTEN_SS(2); else CLUSTEN_SS(1);
#undef CLUSTEN_SS
    note_launch();
    return check_launch();
}

}  // namespace

#define CLUSTEN_DISPATCH(dtype, FN, ...)                                         \
    switch (dtype) {                                                             \
        case CLUSTEN_F32: return FN<float>(__VA_ARGS__);                         \
        case CLUSTEN_F16: return FN<__half>(__VA_ARGS__);                        \
        case CLUSTEN_BF16: return FN<__nv_bfloat16>(__VA_ARGS__);                \
        case CLUSTEN_F64: return FN<double>(__VA_ARGS__);                        \
        default: return CLUSTEN_ERR_DTYPE;                                       \
    }

int launch_gather_sum(const char* label, int dtype, const void* W, const void* X, const int64_t* idx, void* out, int nb, int heads,
                      int n_rows, int n_src, int m, int ic, int c, cudaStream_t s) {
    CLUSTEN_DISPATCH(dtype, gather_sum_t, label, W, X, idx, out, nb, heads, n_rows, n_src, m, ic, c, s)
}

int launch_gather_dot(const char* label, int dtype, const void* X, const void* Y, const int64_t* idx, void* out, int nb, int heads,
                      int n_rows, int n_src, int m, int ic, int c, cudaStream_t s) {
    CLUSTEN_DISPATCH(dtype, gather_dot_t, label, X, Y, idx, out, nb, heads, n_rows, n_src, m, ic, c, s)
}

int launch_scatter_sum(const char* label, int dtype, const void* W, const void* X, const int64_t* idx, const InverseView& inv,
                       void* out, int nb, int heads, int n_rows, int n_tgt, int m, int ic, int c,
                       cudaStream_t s) {
    CLUSTEN_DISPATCH(dtype, scatter_sum_t, label, W, X, idx, inv, out, nb, heads, n_rows, n_tgt, m, ic, c, s)
}

}  // namespace clusten
