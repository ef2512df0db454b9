// Tiled CLUSTEN kernels (declarations; tiled_fwd.cu: QK / AV, wf_tiled.cu: WF).
#pragma once
#include "common.cuh"

namespace clusten {

// Element strides of the operands the gather kernels read through views: X (the gathered rows: key / value)
// and, for the dot product, Y (the tile's own rows: query / d_feat).  Rows themselves are contiguous (32
// elements).  Zero-initialised = the contiguous [b, h, n, 32] layout.
struct GatherStrides {
    long long x_batch, x_head, x_row;
    long long y_batch, y_head, y_row;
};

// gather-sum:  out[b,h,i,:] = sum_j W[b,h,i,j] * X[b,h,idx[b,i,j],:]      (AV forward, d_query)
bool tiled_sum_supported(int dtype, const void* W, const void* X, const void* out, int n, int m, int c);
int launch_tiled_sum(const char* label, int dtype, const void* W, const void* X, const int64_t* idx, void* out, int b, int h, int n,
                     int m, cudaStream_t s, const GatherStrides& gs = GatherStrides{});

// gather-dot:  out[b,h,i,j] = <X[b,h,idx[b,i,j],:], Y[b,h,i,:]>           (QK forward, d_attn)
bool tiled_dot_supported(int dtype, const void* Y, const void* X, const void* out, int n, int m, int c);
int launch_tiled_dot(const char* label, int dtype, const void* X, const void* Y, const int64_t* idx, void* out, int b, int h, int n,
                     int m, cudaStream_t s, const GatherStrides& gs = GatherStrides{});

// fused local attention forward (fused_attn.cu): scores + bias + mask + blank token + softmax + output
bool fused_attention_supported(int dtype, int n, int m, int c);
int launch_fused_attention(int dtype, const void* q, const void* k, const void* v, const int64_t* idx, const void* bias,
                           const void* table, const int64_t* pe_idx, int table_rows, const int64_t* mask,
                           const void* blank_k, const void* blank_v, void* out, int b, int h, int n, int m,
                           GatherStrides gs, cudaStream_t s);

// scatter-sum: out[b,h,t,:] = sum_{idx[b,i,j]==t} W[b,h,i,j] * X[b,h,i,:]   (d_key, d_value)
bool tiled_scatter_supported(int dtype, const void* W, const void* X, const void* out, int n, int m, int c);
int launch_tiled_scatter(const char* label, int dtype, const void* W, const void* X, const int64_t* idx, const InverseView& inv,
                         void* out, int b, int h, int n, int m, cudaStream_t s);

// the structured tiles of the same reduction (scatter_struct.cu); launch_tiled_scatter calls it first
int launch_struct_scatter(const char* label, int dtype, const void* W, const void* X, const InverseView& inv, void* out,
                          int b, int h, int n, int m, cudaStream_t s);

// scatter-sum for WF:  out[b,t,:] = sum_{idx[b,i,j]==t} sum_k W[b,i,j,k] * X[b,i,k,:]   (d_feat)
bool tiled_wf_scatter_supported(int dtype, const void* W, const void* X, const void* out, int n_out, int n, int m,
                                int ic, int c);
int launch_tiled_wf_scatter(const char* label, int dtype, const void* W, const void* X, const int64_t* idx,
                            const InverseView& inv, void* out, int b, int n_out, int n, int m, int ic, int c,
                            cudaStream_t s);

// WF gather side, tiles of 8 rows taken in row_order (nullptr = storage order)
size_t wf_order_bytes(int b, int n_out);
int launch_wf_order(const int64_t* idx, int b, int n_out, int m, int* order, cudaStream_t s);
bool tiled_wf_gather_supported(int dtype, const void* W, const void* F, const void* O, int n_out, int n, int m,
                               int ic, int c);
int launch_tiled_wf_dot(const char* label, int dtype, const void* F, const void* G, const int64_t* idx,
                        const int* order, void* d_weights, int b, int n_out, int n, int m, int ic, int c,
                        cudaStream_t s);
int launch_tiled_wf_sum(const char* label, int dtype, const void* W, const void* F, const int64_t* idx,
                        const int* order, void* out, int b, int n_out, int n, int m, int ic, int c, cudaStream_t s);

// WF d_feat on 8-target tiles with the ic gradient rows of a merge row staged side by side
bool tiled_wf_dfeat_supported(int dtype, const void* W, const void* G, const void* out, int n_out, int n, int m,
                              int ic, int c);
int launch_tiled_wf_dfeat(const char* label, int dtype, const void* W, const void* G, const int64_t* idx,
                          const InverseView& inv, void* d_feat, int b, int n_out, int n, int m, int ic, int c,
                          cudaStream_t s);

// WF forward as a plain walk over the neighbours, half a warp per merge row (wf_direct.cu)
bool wf_forward_direct_supported(int dtype, int n_out, int n, int m, int ic, int c);
int launch_wf_forward_direct(const char* label, int dtype, const void* W, const void* F, const int64_t* idx,
                             const int* order, void* out, int b, int n_out, int n, int m, int ic, int c,
                             cudaStream_t s);
// d_weights for fp32 inputs and ic = 4 the same way
int launch_wf_dweights_direct(const char* label, const void* F, const void* G, const int64_t* idx, const int* order,
                              void* d_weights, int b, int n_out, int n, int m, int c, cudaStream_t s);

}  // namespace clusten
