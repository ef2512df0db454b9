// Merge weights of ClusterMerging in one pass.
//
// Before it calls CLUSTENWF the reference builds the weights of every (merge centre, neighbour) pair from
// three lookups (models/aff_transformer.py:340-358):
//
//     weights[b, i, j, :] = weights_table[pe_idx[b, i, j], :] * (learned_prob[b, nbhd_idx[b, i, j]] * mask[b, i, j])
//
// as a gather of ic-wide table rows over b * n_out * m int64 indices, a gather of the importance scores, and
// two or three elementwise products, each a full pass over a [b, n_out, m, ic] tensor.  Here a thread owns one
// pair: it reads its three 8-byte indices (coalesced), the score and the table row (both from L1 / L2: the
// table is 12321 x ic, the scores b x n) and writes the ic weights once.  The products are formed in fp32 in the
// reference's order -- (score * mask) first, then the table row times that -- and rounded to the output type
// once, which is what the reference's tensors hold when table and scores share a dtype.
#include "tile_core.cuh"

namespace clusten {
namespace {

constexpr int kMergeThreads = 256;

struct MergeParams {
    const void* table;            // [table_rows, ic]
    const int64_t* pe_idx;        // [b, n_out, m]
    const void* prob;             // [b, n] or nullptr (= 1)
    const int64_t* nbhd_idx;      // [b, n_out, m]
    const int64_t* mask;          // [b, n_out, m] or nullptr (= 1)
    void* out;                    // [b, n_out, m, ic]
    long long per_batch;          // n_out * m
    long long pairs;              // b * n_out * m
    int n, ic, table_rows;
};

template <typename T, int ICT>
__global__ void __launch_bounds__(kMergeThreads)
merge_weights_kernel(const MergeParams p) {
    const T* table = static_cast<const T*>(p.table);
    const T* prob = static_cast<const T*>(p.prob);
    T* out = static_cast<T*>(p.out);
    const int ic = ICT > 0 ? ICT : p.ic;
    for (long long z = (long long)blockIdx.x * kMergeThreads + threadIdx.x; z < p.pairs;
         z += (long long)gridDim.x * kMergeThreads) {
        const long long pe = p.pe_idx[z];
        float s = 1.f;
        if (prob) {
            const long long t = p.nbhd_idx[z];
            const long long b = z / p.per_batch;
            s = t >= 0 && t < p.n ? Elem<T>::up(prob[b * p.n + t]) : 0.f;
        }
        if (p.mask) s = Elem<T>::up(Elem<T>::down(__fmul_rn(s, (float)p.mask[z])));
        const bool have = pe >= 0 && pe < p.table_rows;
        if constexpr (ICT == 4) {
            float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
            if (have) w = ld4(table + pe * 4);
            w.x = __fmul_rn(w.x, s);  w.y = __fmul_rn(w.y, s);  w.z = __fmul_rn(w.z, s);  w.w = __fmul_rn(w.w, s);
            st4(out + z * 4, w);
        } else {
            for (int k = 0; k < ic; ++k) {
                const float w = have ? Elem<T>::up(table[pe * ic + k]) : 0.f;
                out[z * ic + k] = Elem<T>::down(__fmul_rn(w, s));
            }
        }
    }
}

template <typename T>
int merge_weights_t(const MergeParams& p, cudaStream_t s) {
    const long long want = (p.pairs + kMergeThreads - 1) / kMergeThreads;
    const long long cap = (long long)sm_count() * 32;
    const int grid = (int)(want < cap ? want : cap);
    const bool vec = p.ic == 4 && reinterpret_cast<uintptr_t>(p.table) % (4 * sizeof(T)) == 0 &&
                     reinterpret_cast<uintptr_t>(p.out) % (4 * sizeof(T)) == 0;
    ScopedKernelTimer timer("merge_weights", s);
    if (vec) merge_weights_kernel<T, 4><<<grid, kMergeThreads, 0, s>>>(p);
    else merge_weights_kernel<T, 0><<<grid, kMergeThreads, 0, s>>>(p);
    note_launch();
    return check_launch();
}

}  // namespace

int launch_merge_weights(int dtype, const void* table, const int64_t* pe_idx, const void* prob, const int64_t* nbhd_idx,
                         const int64_t* mask, void* out, int b, int n_out, int n, int m, int ic, int table_rows,
                         cudaStream_t s) {
    MergeParams p{};
    p.table = table;  p.pe_idx = pe_idx;  p.prob = prob;  p.nbhd_idx = nbhd_idx;  p.mask = mask;  p.out = out;
    p.per_batch = (long long)n_out * m;  p.pairs = p.per_batch * b;
    p.n = n;  p.ic = ic;  p.table_rows = table_rows;
    switch (dtype) {
        case CLUSTEN_F32: return merge_weights_t<float>(p, s);
        case CLUSTEN_F16: return merge_weights_t<__half>(p, s);
        case CLUSTEN_BF16: return merge_weights_t<__nv_bfloat16>(p, s);
        default: return CLUSTEN_ERR_DTYPE;
    }
}

}  // namespace clusten
