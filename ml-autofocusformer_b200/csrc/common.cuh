// Shared device/host helpers of libclusten_b200: element-type traits, vector
// loads, the inverse-index layout and the launch bookkeeping.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/clusten_b200.h"

namespace clusten {

// ---------------------------------------------------------------- element types
template <typename T> struct Elem;
template <> struct Elem<float> {
    using acc_t = float;
    static __device__ __forceinline__ float up(float x) { return x; }
    static __device__ __forceinline__ float down(float x) { return x; }
};
template <> struct Elem<double> {
    using acc_t = double;
    static __device__ __forceinline__ double up(double x) { return x; }
    static __device__ __forceinline__ double down(double x) { return x; }
};
template <> struct Elem<__half> {
    using acc_t = float;
    static __device__ __forceinline__ float up(__half x) { return __half2float(x); }
    static __device__ __forceinline__ __half down(float x) { return __float2half_rn(x); }
};
template <> struct Elem<__nv_bfloat16> {
    using acc_t = float;
    static __device__ __forceinline__ float up(__nv_bfloat16 x) { return __bfloat162float(x); }
    static __device__ __forceinline__ __nv_bfloat16 down(float x) { return __float2bfloat16_rn(x); }
};

// V consecutive elements moved with one load/store instruction.
template <typename T, int V> struct alignas(sizeof(T) * V) Vec { T v[V]; };

template <typename T, int V>
__device__ __forceinline__ Vec<T, V> ldg_vec(const T* p) {
    return *reinterpret_cast<const Vec<T, V>*>(p);
}
template <typename T, int V>
__device__ __forceinline__ void st_vec(T* p, const Vec<T, V>& x) {
    *reinterpret_cast<Vec<T, V>*>(p) = x;
}

// ---------------------------------------------------------------- inverse index
// Layout of the buffer filled by clusten_inverse_build (all int32):
//   [0, 64)                       header: magic, b, n_rows, m, n_targets, #out-of-range indices
//   rowptr  [b][n_targets + 1]    segment start of target t inside its batch element's entries
//   seglen  [b][n_targets]        entries in the segment (<= rowptr[t+1]-rowptr[t])
//   entries [b][n_rows * m]       row * m + slot of one (row, slot) with nbhd_idx == t.
//   tileflag [b][1 + ceil(n_targets / 8)]   [0]: which build handled the batch element (kBuild*);
//                                 [1 + i]: structure of the tile of targets 8i .. 8i+7 (kTile*)
//   (n_targets > kInvSmemTargets only)  scratch [b][3 * n_targets]  counters of the build
// A target that occurs several times in one row gets ONE entry, row * m with
// kDupFlag set; the consumer then scans that row of nbhd_idx for all its
// slots.  Segments are ordered by row, so every reduction order is fixed.
//
// Tile structures (recorded by the structured build, inverse_struct.cu; the general build writes
// kTileGeneral everywhere):
//   kTileRuns      the 8 targets are named by the same rows, once each, target q at slot j0 + q: their
//                  segments have one length and entry k of target q is entry k of target 0 plus q
//   kTileClusters  every segment consists of whole clusters: entries 8k .. 8k+7 are the rows 8c .. 8c+7
//                  at one slot; no row names a target twice; at most kStructMaxPairs (cluster, slot)
//                  pairs in the tile
constexpr int kInvHeaderInts = 64;
constexpr uint32_t kInvMagic = 0x434c5354u;
constexpr uint32_t kDupFlag = 0x80000000u;
constexpr int kBuildGeneral = 0, kBuildRuns = 1, kBuildClusters = 2;
constexpr int kTileGeneral = 0, kTileRuns = 1, kTileClusters = 2;
constexpr int kStructMaxPairs = 96;
constexpr int kInvSmemTargets = 18000;       // up to here the build keeps its per-target counters in shared memory
constexpr int kInvMaxTargets = 1 << 20;      // beyond kInvSmemTargets they live behind the entries, in the buffer itself

struct InverseView {
    const int* rowptr;    // [b][nt + 1]
    const int* seglen;    // [b][nt]
    const int* entries;   // [b][n_rows * m]
    const int* tileflag;  // [b][1 + ntiles]
    int ntiles;           // ceil(nt / 8)
};

__host__ __device__ inline int inverse_tiles(int nt) { return (nt + 7) / 8; }

__host__ __device__ inline size_t inv_align(size_t x) { return (x + 63) & ~size_t(63); }

// counters of the build when they do not fit in shared memory: [b][3 * nt] behind the entries
inline size_t inverse_scratch_ints(int b, int nt) {
    return nt > kInvSmemTargets ? inv_align(size_t(b) * 3 * nt) : 0;
}

inline size_t inverse_ints(int b, int n_rows, int m, int nt) {
    return kInvHeaderInts + inv_align(size_t(b) * (nt + 1)) + inv_align(size_t(b) * nt) +
           inv_align(size_t(b) * n_rows * m) + inv_align(size_t(b) * (1 + inverse_tiles(nt))) +
           inverse_scratch_ints(b, nt);
}

inline InverseView inverse_view(const void* buf, int b, int n_rows, int m, int nt) {
    const int* p = static_cast<const int*>(buf);
    InverseView v;
    v.rowptr = p + kInvHeaderInts;
    v.seglen = v.rowptr + inv_align(size_t(b) * (nt + 1));
    v.entries = v.seglen + inv_align(size_t(b) * nt);
    v.tileflag = v.entries + inv_align(size_t(b) * n_rows * m);
    v.ntiles = inverse_tiles(nt);
    return v;
}

// ---------------------------------------------------------------- launches
void note_launch();               // counts one kernel launch (api.cu)

// Brackets one kernel launch with CUDA events when timing is enabled (api.cu).
struct ScopedKernelTimer {
    ScopedKernelTimer(const char* name, cudaStream_t s);
    ~ScopedKernelTimer();
    int slot;
    cudaStream_t stream;
};
int check_launch();               // cudaGetLastError -> CLUSTEN_OK / CLUSTEN_ERR_CUDA
// CLUSTEN_SPLIT_TIMING=1 in the environment: kernels that share an operator's timing label (the structured
// and the general part of one reduction) are timed under names of their own
bool split_timing_labels();
int sm_count();                   // multiprocessors of the current device (cached per device)
// One-time set-up of a kernel on the current device: raises its dynamic shared-memory limit to
// smem bytes and returns how many CTAs of `threads` threads fit on one multiprocessor (>= 1), or a
// negative status.  The answer is cached per (kernel, device, smem), so repeated launches cost a
// map lookup instead of two runtime calls.
int resident_ctas(const void* kernel, int threads, size_t smem);

template <typename T> struct DtypeOf;
template <> struct DtypeOf<float> { static constexpr int value = CLUSTEN_F32; };
template <> struct DtypeOf<__half> { static constexpr int value = CLUSTEN_F16; };
template <> struct DtypeOf<__nv_bfloat16> { static constexpr int value = CLUSTEN_BF16; };
template <> struct DtypeOf<double> { static constexpr int value = CLUSTEN_F64; };

inline int dtype_size(int dtype) {
    switch (dtype) {
        case CLUSTEN_F32: return 4;
        case CLUSTEN_F16: return 2;
        case CLUSTEN_BF16: return 2;
        case CLUSTEN_F64: return 8;
        default: return 0;
    }
}

// ---------------------------------------------------------------- generic kernels (generic.cu)
// out[bb, row, ic, :] = sum_j W[bb, row, j, ic] * X[bb, idx[bb / heads, row, j], :]
int launch_gather_sum(const char* label, int dtype, const void* W, const void* X, const int64_t* idx, void* out,
                      int nb, int heads, int n_rows, int n_src, int m, int ic, int c, cudaStream_t s);
// out[bb, row, j, ic] = sum_c X[bb, idx[bb / heads, row, j], c] * Y[bb, row, ic, c]
int launch_gather_dot(const char* label, int dtype, const void* X, const void* Y, const int64_t* idx, void* out,
                      int nb, int heads, int n_rows, int n_src, int m, int ic, int c, cudaStream_t s);
// out[bb, t, :] = sum_{(row, j): idx[bb / heads, row, j] == t} sum_ic W[bb, row, j, ic] * X[bb, row, ic, :]
int launch_scatter_sum(const char* label, int dtype, const void* W, const void* X, const int64_t* idx, const InverseView& inv,
                       void* out, int nb, int heads, int n_rows, int n_tgt, int m, int ic, int c,
                       cudaStream_t s);

// api.cu: every argument check of clusten_av_backward (sizes, dtype, pointers and their alignment)
int validate_av_backward(const void* d_feat, const void* attn, const void* value, const int64_t* nbhd_idx,
                         const void* inverse, const void* d_attn, const void* d_value, int b, int h, int n, int m,
                         int c, int dtype);

// knn.cu
int launch_knn2d(const float* query, const float* db, int b, int nq, int n, int k, int64_t* idx_out, float* dist_out,
                 cudaStream_t s);

// nbhd.cu
int launch_nbhd_build(const float* pos, const int64_t* member_idx, const int64_t* cluster_mask,
                      const int64_t* nearest_cluster, int64_t* nbhd_idx, int64_t* nbhd_mask, int64_t* pe_idx, int b,
                      int n, int k, int cs, int nnc, int rel_pos_width, int table_width, cudaStream_t s);

// merge.cu
int launch_merge_weights(int dtype, const void* table, const int64_t* pe_idx, const void* prob, const int64_t* nbhd_idx,
                         const int64_t* mask, void* out, int b, int n_out, int n, int m, int ic, int table_rows,
                         cudaStream_t s);

// inverse.cu
int launch_inverse_build(const int64_t* idx, int b, int n_rows, int m, int nt, void* buf, cudaStream_t s);
// inverse_struct.cu: the build for cluster- and run-structured tables; runs first, marks what it handled
int launch_inverse_struct(const int64_t* idx, int b, int n_rows, int m, int nt, void* buf, cudaStream_t s);

}  // namespace clusten
