/*
 * clusten_oracle.c -- CPU restatement of the reference's eight CLUSTEN kernels.
 *
 * TEST INFRASTRUCTURE ONLY: the checker for tests/, __graft_entry__.smoke() and
 * the cpu_baseline leg of bench.py.  Nothing the product ships calls it.
 *
 * Each function follows one kernel of apple/ml-autofocusformer (clusten/src/*.cu,
 * path:line given at the function): same index arithmetic, same loop nest, and
 * the same accumulation type as the reference (it accumulates in the tensor's
 * scalar type: clustenqk_cuda_kernel.cu:40).  The scatter gradients are summed
 * in (row, slot) order, one of the orders the reference's atomicAdd may take.
 * Built for float (suffix _f32) and double (_f64); the double build fed with
 * fp32 / bf16-rounded inputs is the "exact" answer the tolerances refer to.
 *
 * Parity pin: checked against outputs of the reference's own CUDA extension
 * (built unmodified by oracle/build_ref.py, run on a B200) stored in
 * tests/golden/ref_cuda_*.npz, and against the PyTorch gather formulation of
 * the reference's tests (oracle/formula.py).
 *
 * Layouts (contiguous): q,k,v [b,h,n,c]; attn [b,h,n,m]; idx int64 [b,n,m];
 * weights [b,n_,m,ic]; feat [b,n,c]; feat_new [b,n_,ic,c].
 * Build:  gcc -O2 -fopenmp -shared -fPIC -o oracle/_build/libclusten_oracle.so oracle/clusten_oracle.c
 */
#include <stdint.h>
#include <string.h>

#define DEFINE_ORACLE(T, SFX)                                                                               \
/* K1 clusten_qk_cuda_forward_kernel, clusten/src/clustenqk_cuda_kernel.cu:18-49.                           \
 * The reference reads a pre-transposed key [b,h,c,n] (clusten/clusten.py:30); here key is [b,h,n,c]. */    \
void oracle_qk_forward_##SFX(const T* q, const T* k, const int64_t* idx, T* attn,                           \
                             int b, int h, int n, int m, int c) {                                           \
    _Pragma("omp parallel for collapse(2) schedule(static)")                                                \
    for (int z = 0; z < b * h; ++z)                                                                         \
        for (int i = 0; i < n; ++i) {                                                                       \
            const int bi = z / h;                                                                           \
            const T* qr = q + ((size_t)z * n + i) * c;                                                      \
            for (int ni = 0; ni < m; ++ni) {                                                                \
                const int64_t nbi = idx[((size_t)bi * n + i) * m + ni];                                     \
                const T* kr = k + ((size_t)z * n + nbi) * c;                                                \
                T updt = 0;                                                                                 \
                for (int cc = 0; cc < c; ++cc) updt += qr[cc] * kr[cc];                                     \
                attn[((size_t)z * n + i) * m + ni] = updt;                                                  \
            }                                                                                               \
        }                                                                                                   \
}                                                                                                           \
/* K2 clusten_qk_cuda_backward_kernel, clustenqk_cuda_kernel.cu:91-132 (d_key zero-filled at :152). */      \
void oracle_qk_backward_##SFX(const T* d_attn, const T* q, const T* k, const int64_t* idx,                  \
                              T* d_q, T* d_k, int b, int h, int n, int m, int c) {                          \
    memset(d_k, 0, sizeof(T) * (size_t)b * h * n * c);                                                      \
    _Pragma("omp parallel for schedule(static)")                                                            \
    for (int z = 0; z < b * h; ++z) {                                                                       \
        const int bi = z / h;                                                                               \
        for (int i = 0; i < n; ++i)                                                                         \
            for (int cc = 0; cc < c; ++cc) {                                                                \
                T dq_update = 0;                                                                            \
                for (int ni = 0; ni < m; ++ni) {                                                            \
                    const int64_t nbi = idx[((size_t)bi * n + i) * m + ni];                                 \
                    const T da = d_attn[((size_t)z * n + i) * m + ni];                                      \
                    dq_update += k[((size_t)z * n + nbi) * c + cc] * da;                                    \
                    d_k[((size_t)z * n + nbi) * c + cc] += q[((size_t)z * n + i) * c + cc] * da;            \
                }                                                                                           \
                d_q[((size_t)z * n + i) * c + cc] = dq_update;                                              \
            }                                                                                               \
    }                                                                                                       \
}                                                                                                           \
/* K3 clusten_av_cuda_forward_kernel, clusten/src/clustenav_cuda_kernel.cu:18-50. */                        \
void oracle_av_forward_##SFX(const T* attn, const T* v, const int64_t* idx, T* feat,                        \
                             int b, int h, int n, int m, int c) {                                           \
    _Pragma("omp parallel for collapse(2) schedule(static)")                                                \
    for (int z = 0; z < b * h; ++z)                                                                         \
        for (int i = 0; i < n; ++i) {                                                                       \
            const int bi = z / h;                                                                           \
            for (int cc = 0; cc < c; ++cc) {                                                                \
                T updt = 0;                                                                                 \
                for (int ni = 0; ni < m; ++ni) {                                                            \
                    const int64_t nbi = idx[((size_t)bi * n + i) * m + ni];                                 \
                    updt += attn[((size_t)z * n + i) * m + ni] * v[((size_t)z * n + nbi) * c + cc];         \
                }                                                                                           \
                feat[((size_t)z * n + i) * c + cc] = updt;                                                  \
            }                                                                                               \
        }                                                                                                   \
}                                                                                                           \
/* K4 clusten_av_cuda_backward_kernel :93-127 (d_v) and K5 clusten_av_attn_cuda_backward_kernel :129-160. */\
void oracle_av_backward_##SFX(const T* d_feat, const T* attn, const T* v, const int64_t* idx,               \
                              T* d_attn, T* d_v, int b, int h, int n, int m, int c) {                       \
    memset(d_v, 0, sizeof(T) * (size_t)b * h * n * c);                                                      \
    _Pragma("omp parallel for schedule(static)")                                                            \
    for (int z = 0; z < b * h; ++z) {                                                                       \
        const int bi = z / h;                                                                               \
        for (int i = 0; i < n; ++i)                                                                         \
            for (int ni = 0; ni < m; ++ni) {                                                                \
                const int64_t nbi = idx[((size_t)bi * n + i) * m + ni];                                     \
                const T a = attn[((size_t)z * n + i) * m + ni];                                             \
                T updt = 0;                                                                                 \
                for (int cc = 0; cc < c; ++cc) {                                                            \
                    const T df = d_feat[((size_t)z * n + i) * c + cc];                                      \
                    updt += v[((size_t)z * n + nbi) * c + cc] * df;                                         \
                    d_v[((size_t)z * n + nbi) * c + cc] += df * a;                                          \
                }                                                                                           \
                d_attn[((size_t)z * n + i) * m + ni] = updt;                                                \
            }                                                                                               \
    }                                                                                                       \
}                                                                                                           \
/* K6 clusten_wf_cuda_forward_kernel, clusten/src/clustenwf_cuda_kernel.cu:18-53. */                        \
void oracle_wf_forward_##SFX(const T* w, const T* feat, const int64_t* idx, T* feat_new,                    \
                             int b, int n_out, int n, int m, int ic, int c) {                               \
    _Pragma("omp parallel for collapse(2) schedule(static)")                                                \
    for (int bi = 0; bi < b; ++bi)                                                                          \
        for (int i = 0; i < n_out; ++i)                                                                     \
            for (int cc = 0; cc < c; ++cc)                                                                  \
                for (int k = 0; k < ic; ++k) {                                                              \
                    T updt = 0;                                                                             \
                    for (int ni = 0; ni < m; ++ni) {                                                        \
                        const int64_t nbi = idx[((size_t)bi * n_out + i) * m + ni];                         \
                        updt += w[(((size_t)bi * n_out + i) * m + ni) * ic + k] *                           \
                                feat[((size_t)bi * n + nbi) * c + cc];                                      \
                    }                                                                                       \
                    feat_new[(((size_t)bi * n_out + i) * ic + k) * c + cc] = updt;                          \
                }                                                                                           \
}                                                                                                           \
/* K7 clusten_wf_cuda_backward_kernel :96-135 (d_feat) and K8 clusten_wf_weights_cuda_backward_kernel       \
 * :137-169 (d_weights). */                                                                                 \
void oracle_wf_backward_##SFX(const T* d_feat_new, const T* w, const T* feat, const int64_t* idx,           \
                              T* d_w, T* d_feat, int b, int n_out, int n, int m, int ic, int c) {           \
    memset(d_feat, 0, sizeof(T) * (size_t)b * n * c);                                                       \
    _Pragma("omp parallel for schedule(static)")                                                            \
    for (int bi = 0; bi < b; ++bi)                                                                          \
        for (int i = 0; i < n_out; ++i)                                                                     \
            for (int ni = 0; ni < m; ++ni) {                                                                \
                const int64_t nbi = idx[((size_t)bi * n_out + i) * m + ni];                                 \
                for (int cc = 0; cc < c; ++cc) {                                                            \
                    T updt = 0;                                                                             \
                    for (int k = 0; k < ic; ++k)                                                            \
                        updt += d_feat_new[(((size_t)bi * n_out + i) * ic + k) * c + cc] *                  \
                                w[(((size_t)bi * n_out + i) * m + ni) * ic + k];                            \
                    d_feat[((size_t)bi * n + nbi) * c + cc] += updt;                                        \
                }                                                                                           \
                for (int k = 0; k < ic; ++k) {                                                              \
                    T updt = 0;                                                                             \
                    for (int cc = 0; cc < c; ++cc)                                                          \
                        updt += feat[((size_t)bi * n + nbi) * c + cc] *                                     \
                                d_feat_new[(((size_t)bi * n_out + i) * ic + k) * c + cc];                   \
                    d_w[(((size_t)bi * n_out + i) * m + ni) * ic + k] = updt;                               \
                }                                                                                           \
            }                                                                                               \
}

DEFINE_ORACLE(float, f32)
DEFINE_ORACLE(double, f64)
