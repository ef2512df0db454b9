// Neighbourhood tables of a stage, built in one pass.
//
// AutoFocusFormer gives every token the members of its nnc nearest clusters as neighbours and looks the
// position bias up by the neighbour's offset (models/aff_transformer.py:476-487 of the reference):
//
//     c = nearest_cluster[b, i, r]          r < nnc
//     t = member_idx[b, c, s]               s < cs,   slot j = r * cs + s
//     nbhd_idx[b, i, j]  = t
//     nbhd_mask[b, i, j] = cluster_mask[b, c, s]                          (when there is a mask)
//     rel                = pos[b, t] - (pos[b, i] - rel_pos_width)          (fp32, both coordinates)
//     pe_idx[b, i, j]    = (int64)(rel.y * table_width + rel.x)             (fp32 product and sum, truncated)
//
// The reference does this with three gathers and four elementwise kernels over [b, n, nnc * cs] tensors;
// here a thread owns one (token, nearest cluster) pair and writes its cs consecutive slots of the two or
// three outputs, 64 contiguous bytes each for cs = 8, so that a warp writes 2 KB runs.  The tables it
// reads (positions, cluster members) are small and stay in L1 / L2: the kernel is bound by its writes.
#include "common.cuh"

namespace clusten {
namespace {

constexpr int kNbhdThreads = 256;

struct NbhdParams {
    const float2* pos;            // [b, n]
    const int64_t* member;        // [b, k, cs]
    const int64_t* cmask;         // [b, k, cs] or nullptr
    const int64_t* nearest;       // [b, n, nnc]
    int64_t* nbhd_idx;            // [b, n, nnc * cs]
    int64_t* nbhd_mask;           // [b, n, nnc * cs] or nullptr
    int64_t* pe_idx;              // [b, n, nnc * cs]
    int n, k, cs, nnc;
    float width, table;           // rel_pos_width, table_width
    long long pairs;              // b * n * nnc
};

__device__ __forceinline__ long long pe_of(float2 pt, float2 base, float table) {
    const float rx = __fsub_rn(pt.x, base.x), ry = __fsub_rn(pt.y, base.y);
    return (long long)__fadd_rn(__fmul_rn(ry, table), rx);
}

template <int CS>
__global__ void __launch_bounds__(kNbhdThreads)
nbhd_build_kernel(const NbhdParams p) {
    const int cs = CS > 0 ? CS : p.cs;
    for (long long z = (long long)blockIdx.x * kNbhdThreads + threadIdx.x; z < p.pairs;
         z += (long long)gridDim.x * kNbhdThreads) {
        const long long tok = z / p.nnc;                          // b * n + i
        const int b = (int)(tok / p.n);
        const long long c = p.nearest[z];
        const bool have = c >= 0 && c < p.k;                      // a cluster id out of range names nobody
        const int64_t* mrow = p.member + ((long long)b * p.k + (have ? c : 0)) * cs;
        const int64_t* krow = p.cmask ? p.cmask + ((long long)b * p.k + (have ? c : 0)) * cs : nullptr;
        const float2 self = p.pos[tok];
        const float2 base = make_float2(__fsub_rn(self.x, p.width), __fsub_rn(self.y, p.width));
        const float2* posb = p.pos + (long long)b * p.n;
        int64_t* oi = p.nbhd_idx + z * cs;
        int64_t* op = p.pe_idx + z * cs;
        int64_t* om = p.nbhd_mask ? p.nbhd_mask + z * cs : nullptr;
        if constexpr (CS == 8) {
            longlong2 t[4], pe[4];
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                t[v] = have ? reinterpret_cast<const longlong2*>(mrow)[v] : make_longlong2(-1, -1);
            }
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const bool okx = t[v].x >= 0 && t[v].x < p.n, oky = t[v].y >= 0 && t[v].y < p.n;
                const float2 px = okx ? posb[t[v].x] : base, py = oky ? posb[t[v].y] : base;
                pe[v].x = okx ? pe_of(px, base, p.table) : 0;
                pe[v].y = oky ? pe_of(py, base, p.table) : 0;
            }
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                reinterpret_cast<longlong2*>(oi)[v] = t[v];
                reinterpret_cast<longlong2*>(op)[v] = pe[v];
            }
            if (om) {
#pragma unroll
                for (int v = 0; v < 4; ++v)
                    reinterpret_cast<longlong2*>(om)[v] =
                        have ? reinterpret_cast<const longlong2*>(krow)[v] : make_longlong2(0, 0);
            }
        } else {
            for (int s = 0; s < cs; ++s) {
                const long long t = have ? mrow[s] : -1;
                const bool ok = t >= 0 && t < p.n;
                oi[s] = t;
                op[s] = ok ? pe_of(posb[t], base, p.table) : 0;
                if (om) om[s] = have ? krow[s] : 0;
            }
        }
    }
}

}  // namespace

int launch_nbhd_build(const float* pos, const int64_t* member_idx, const int64_t* cluster_mask,
                      const int64_t* nearest_cluster, int64_t* nbhd_idx, int64_t* nbhd_mask, int64_t* pe_idx, int b,
                      int n, int k, int cs, int nnc, int rel_pos_width, int table_width, cudaStream_t s) {
    NbhdParams p{};
    p.pos = reinterpret_cast<const float2*>(pos);
    p.member = member_idx;  p.cmask = cluster_mask;  p.nearest = nearest_cluster;
    p.nbhd_idx = nbhd_idx;  p.nbhd_mask = nbhd_mask;  p.pe_idx = pe_idx;
    p.n = n;  p.k = k;  p.cs = cs;  p.nnc = nnc;
    p.width = (float)rel_pos_width;  p.table = (float)table_width;
    p.pairs = (long long)b * n * nnc;
    const long long want = (p.pairs + kNbhdThreads - 1) / kNbhdThreads;
    const long long cap = (long long)sm_count() * 32;
    const int grid = (int)(want < cap ? want : cap);
    // rows of 8 int64 are copied 16 bytes at a time
    auto a16 = [](const void* q) { return q == nullptr || reinterpret_cast<uintptr_t>(q) % 16 == 0; };
    const bool vec = cs == 8 && a16(member_idx) && a16(cluster_mask) && a16(nbhd_idx) && a16(nbhd_mask) && a16(pe_idx);
    ScopedKernelTimer timer("nbhd_build", s);
    if (vec) nbhd_build_kernel<8><<<grid, kNbhdThreads, 0, s>>>(p);
    else nbhd_build_kernel<0><<<grid, kNbhdThreads, 0, s>>>(p);
    note_launch();
    return check_launch();
}

}  // namespace clusten
