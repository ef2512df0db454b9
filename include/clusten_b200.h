/*
 * clusten_b200.h -- C ABI of libclusten_b200.so
 *
 * B200 (sm_100a) implementation of AutoFocusFormer's CLUSTEN neighbourhood
 * operators.  Every entry point takes plain device pointers and sizes, is
 * asynchronous on the given CUDA stream, allocates nothing and returns a
 * status code (0 = CLUSTEN_OK, negative = error, see clusten_status_string).
 *
 * Each function names the interface of apple/ml-autofocusformer that it
 * replaces (path inside that project : line).
 *
 * Tensor layouts are the reference's, contiguous, last dimension fastest:
 *   query/key/value/d_query/d_key/d_value/feat_out(AV)   [b, h, n, c]
 *   attn / d_attn                                       [b, h, n, m]
 *   nbhd_idx (QK, AV)                                   [b, n, m]    int64, values in [0, n)
 *   weights / d_weights (WF)                            [b, n_, m, ic]
 *   feat / d_feat (WF)                                  [b, n, c]
 *   nbhd_idx (WF)                                       [b, n_, m]   int64, values in [0, n)
 *   feat_new / d_feat_new (WF)                          [b, n_, ic, c]
 * An index outside [0, n) is never dereferenced: the neighbour contributes
 * zero (forward, gather-side gradients) and receives nothing (scatter-side
 * gradients).  The reference does not check (clusten/src/clustenqk_cuda_kernel.cu:38).
 *
 * dtype selects the element type of every floating tensor of a call; sums
 * are accumulated in fp32 (fp64 for CLUSTEN_F64) whatever the element type.
 */
#ifndef CLUSTEN_B200_H_
#define CLUSTEN_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define CLUSTEN_API __attribute__((visibility("default")))
#else
#define CLUSTEN_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* element types: the reference dispatches fp64/fp32/fp16
 * (AT_DISPATCH_FLOATING_TYPES_AND_HALF, clusten/src/clustenqk_cuda_kernel.cu:78);
 * bf16 is an addition. */
enum {
    CLUSTEN_F32 = 0,
    CLUSTEN_F16 = 1,
    CLUSTEN_BF16 = 2,
    CLUSTEN_F64 = 3
};

enum {
    CLUSTEN_OK = 0,
    CLUSTEN_ERR_DTYPE = -1,       /* dtype is not one of the enum above */
    CLUSTEN_ERR_SHAPE = -2,       /* a size is <= 0 or a product overflows int32 */
    CLUSTEN_ERR_NULL = -3,        /* a required pointer is NULL */
    CLUSTEN_ERR_ALIGN = -4,       /* a pointer is not aligned to its element size */
    CLUSTEN_ERR_WORKSPACE = -5,   /* inverse-index or row-order buffer too small or not built for these sizes */
    CLUSTEN_ERR_UNSUPPORTED = -6, /* size outside what the kernels handle (see the function) */
    CLUSTEN_ERR_CUDA = -7,        /* the CUDA runtime reported an error at launch */
    CLUSTEN_ERR_NOALLOC_CAPACITY = -8 /* clusten_av_backward_noalloc: sizes exceed the built-in array */
};

/* Human-readable name of a status code; never NULL. */
CLUSTEN_API const char* clusten_status_string(int status);

/* Library version as major*10000 + minor*100 + patch. */
CLUSTEN_API int clusten_version(void);

/* Number of kernels this library has launched in this process (all threads). */
CLUSTEN_API unsigned long long clusten_launch_count(void);

/* Per-kernel timing for benchmarks.  While enabled, every kernel launch of the
 * library is bracketed by two CUDA events recorded on the launch stream.
 * clusten_timing_collect synchronises those events, writes one line per kernel
 * name, "name launches total_ms\n", into buf (at most buf_bytes - 1 characters,
 * NUL-terminated), clears the record and returns the number of lines, or a
 * negative status.  Timing allocates CUDA events; leave it off in production.
 * No counterpart in the reference. */
CLUSTEN_API int clusten_timing_enable(int on);
CLUSTEN_API int clusten_timing_collect(char* buf, size_t buf_bytes);

/* ------------------------------------------------------------------------
 * Inverse neighbour index.
 *
 * The scatter-side gradients (d_key, d_value, d_feat) are computed as a
 * segmented reduction over, for every target token t, the list of
 * (row, slot) pairs with nbhd_idx[b, row, slot] == t.  This replaces the
 * reference's atomicAdd scatter (clusten/src/clustenqk_cuda_kernel.cu:125,
 * clustenav_cuda_kernel.cu:121, clustenwf_cuda_kernel.cu:129) and makes the
 * gradients bit-reproducible.  One inverse serves every backward call that
 * uses the same nbhd_idx tensor.  The buffer also records, per tile of 8
 * targets, whether the tile has one of the two shapes AutoFocusFormer's tables
 * produce (the 8 tokens of a cluster share a row; or every row is made of whole
 * clusters); the backward entry points use a leaner kernel on such tiles.
 *
 *   n_rows    rows of nbhd_idx per batch element (n for QK/AV, n_ for WF)
 *   n_targets number of tokens the indices point into (n)
 * Limits: m <= 2048, n_targets <= 2^20, n_rows * m < 2^31; otherwise
 * CLUSTEN_ERR_UNSUPPORTED.  Up to 18000 targets the build keeps its per-target
 * counters in shared memory; beyond that they live in the buffer itself (which
 * clusten_inverse_bytes sizes accordingly) and the build is slower.
 * ---------------------------------------------------------------------- */
CLUSTEN_API size_t clusten_inverse_bytes(int b, int n_rows, int m, int n_targets);

CLUSTEN_API int clusten_inverse_build(const int64_t* nbhd_idx, int b, int n_rows, int m, int n_targets,
                          void* inverse, size_t inverse_bytes, void* stream);

/* ------------------------------------------------------------------------
 * QK: attn[b,h,i,j] = sum_c query[b,h,i,c] * key[b,h,nbhd_idx[b,i,j],c]
 * replaces clusten_qk_forward (clusten/src/clustenqk_cuda.cpp:25-33, kernel
 * clustenqk_cuda_kernel.cu:18-49).  key is [b,h,n,c]; the reference's
 * pre-transposed [b,h,c,n] copy (clusten/clusten.py:30) is not needed.
 * ---------------------------------------------------------------------- */
CLUSTEN_API int clusten_qk_forward(const void* query, const void* key, const int64_t* nbhd_idx, void* attn,
                       int b, int h, int n, int m, int c, int dtype, void* stream);

/* QK / AV forward on VIEWS.  The model hands query, key and value as permuted views of its Linear outputs
 * (models/aff_transformer.py:117-119: element strides (n C, c, C, 1) and (n 2C, 2c, 2C, 1) with C = h c), and
 * the reference copies each of them first (clusten/clusten.py:23-24,50).  These two entry points read them
 * in place: *_strides = element strides of (batch, head, row); the c elements of a row are contiguous.
 * attn (input of AV) and all outputs stay contiguous.  Requirements: the shapes of the tiled kernels
 * (c = 32, m <= 48), every pointer and every stride a multiple of 16 bytes; otherwise
 * CLUSTEN_ERR_UNSUPPORTED, and the caller copies and uses the contiguous entry point. */
CLUSTEN_API int clusten_qk_forward_strided(const void* query, const long long* query_strides,
                                           const void* key, const long long* key_strides,
                                           const int64_t* nbhd_idx, void* attn,
                                           int b, int h, int n, int m, int c, int dtype, void* stream);
CLUSTEN_API int clusten_av_forward_strided(const void* attn, const void* value, const long long* value_strides,
                                           const int64_t* nbhd_idx, void* feat,
                                           int b, int h, int n, int m, int c, int dtype, void* stream);

/* Fused local attention, forward only (opt-in; the separate operators above remain the contract):
 *   logits[b,h,i,j] = <query[b,h,i], key[b,h,idx[b,i,j]]> + pos_bias[b,h,i,j]            (pos_bias != NULL)
 *                                                        + pe_table[pe_idx[b,i,j], h]     (pe_table != NULL)
 *                                                        + (1 - mask[b,i,j]) * -100       (mask != NULL)
 *   blank[b,h,i]    = <query[b,h,i], blank_k[h]>                                          (blank_k != NULL)
 *   p = softmax over the m neighbours and the blank token
 *   out[b,h,i,:]    = sum_j p[j] * value[b,h,idx[b,i,j],:] + p[blank] * blank_v[h,:]
 * i.e. the chain of models/aff_transformer.py:120-155 (QK :120, position embedding :129-134, mask :136-137,
 * blank token :140-141, softmax :142, AV :154, blank value :147,155) with the query already scaled (:104); the
 * [b,h,n,m] attention tensor is never written.  query_strides / kv_strides: element strides (batch, head, row)
 * of views with contiguous rows, or NULL for contiguous [b,h,n,c]; key and value share kv_strides (they are
 * the two halves of the model's kv Linear output).  pe_table is [table_rows, h]; mask and pe_idx are int64
 * [b,n,m]; blank_k / blank_v are [h, c].  Shapes of the tiled kernels only (c = 32, m <= 48), pointers of
 * query / key / value / out / blank_* on 16-byte boundaries; otherwise CLUSTEN_ERR_UNSUPPORTED.
 * The reference has no fused counterpart. */
CLUSTEN_API int clusten_local_attention_forward(const void* query, const long long* query_strides,
                                                const void* key, const void* value, const long long* kv_strides,
                                                const int64_t* nbhd_idx,
                                                const void* pos_bias, const void* pe_table, const int64_t* pe_idx,
                                                int table_rows, const int64_t* mask,
                                                const void* blank_k, const void* blank_v, void* out,
                                                int b, int h, int n, int m, int c, int dtype, void* stream);

/* d_query[b,h,i,c] = sum_j key[b,h,idx,c] * d_attn[b,h,i,j]
 * d_key[b,h,t,c]   = sum_{(i,j): idx[b,i,j]==t} query[b,h,i,c] * d_attn[b,h,i,j]
 * replaces clusten_qk_backward (clustenqk_cuda.cpp:35-45, kernel :91-132).
 * inverse: built by clusten_inverse_build(nbhd_idx, b, n, m, n, ...). */
CLUSTEN_API int clusten_qk_backward(const void* d_attn, const void* query, const void* key,
                        const int64_t* nbhd_idx, const void* inverse,
                        void* d_query, void* d_key,
                        int b, int h, int n, int m, int c, int dtype, void* stream);

/* ------------------------------------------------------------------------
 * AV: feat[b,h,i,c] = sum_j attn[b,h,i,j] * value[b,h,nbhd_idx[b,i,j],c]
 * replaces clusten_av_forward (clusten/src/clustenav_cuda.cpp:25-33, kernel
 * clustenav_cuda_kernel.cu:18-50).
 * ---------------------------------------------------------------------- */
CLUSTEN_API int clusten_av_forward(const void* attn, const void* value, const int64_t* nbhd_idx, void* feat,
                       int b, int h, int n, int m, int c, int dtype, void* stream);

/* d_attn[b,h,i,j] = sum_c value[b,h,idx,c] * d_feat[b,h,i,c]
 * d_value[b,h,t,c] = sum_{(i,j): idx[b,i,j]==t} attn[b,h,i,j] * d_feat[b,h,i,c]
 * replaces clusten_av_backward (clustenav_cuda.cpp:35-45, kernels :93-160). */
CLUSTEN_API int clusten_av_backward(const void* d_feat, const void* attn, const void* value,
                        const int64_t* nbhd_idx, const void* inverse,
                        void* d_attn, void* d_value,
                        int b, int h, int n, int m, int c, int dtype, void* stream);

/* AV backward without a workspace argument, for callers that cannot allocate.
 * Same results as clusten_av_backward.  The inverse neighbour index is built, on
 * every call, into an array that is part of the library image on each GPU
 * (CLUSTEN_NOALLOC_MAX_INTS * 4 bytes, held until the process exits); the call
 * makes no cudaMalloc / cudaFree and no allocating library call.  It is meant for
 * hosts that own all device memory themselves or run inside an engine's enqueue
 * callback and so have no buffer to pass and may not ask for one.
 * Limit: clusten_inverse_bytes(b, n, m, n) <= 4 * CLUSTEN_NOALLOC_MAX_INTS, i.e.
 * 64 + roundup64(b * (n + 1)) + roundup64(b * n) + roundup64(b * n * m) + roundup64(b * (1 + ceil(n / 8)))
 * ints, e.g. b = 21, n = 3136, m = 48; larger calls return CLUSTEN_ERR_NOALLOC_CAPACITY.
 * Every argument is checked before anything is launched, so a rejected call leaves the array and the
 * outputs untouched.  The array's address is looked up once per device ordinal and kept for the life of the
 * process: do not use this entry point after cudaDeviceReset.
 * The first call on a device looks up the array's device address (a little set-up
 * work: make that call before any stream capture).  All calls share the array, so
 * calls that overlap on the GPU race; serialise them on one stream.
 * Has no counterpart in the reference. */
#define CLUSTEN_NOALLOC_MAX_INTS 3407936
CLUSTEN_API int clusten_av_backward_noalloc(const void* d_feat, const void* attn, const void* value,
                                            const int64_t* nbhd_idx, void* d_attn, void* d_value,
                                            int b, int h, int n, int m, int c, int dtype, void* stream);

/* ------------------------------------------------------------------------
 * WF: feat_new[b,i,ic,c] = sum_j weights[b,i,j,ic] * feat[b,nbhd_idx[b,i,j],c]
 * replaces clusten_wf_forward (clusten/src/clustenwf_cuda.cpp:25-33, kernel
 * clustenwf_cuda_kernel.cu:18-53).  n_out = n_ (rows of weights / nbhd_idx).
 * ---------------------------------------------------------------------- */
CLUSTEN_API int clusten_wf_forward(const void* weights, const void* feat, const int64_t* nbhd_idx,
                                   const void* row_order, void* feat_new,
                                   int b, int n_out, int n, int m, int ic, int c, int dtype, void* stream);

/* Row order for the WF kernels: a permutation of the n_out rows of every batch
 * element (int32 [b][n_out]) that puts rows with nearby neighbourhoods next to
 * each other, so that one warp's 8 rows share most of the feature rows they
 * gather.  The reference has no such step: its merge centres come out of an
 * unsorted top-k (models/aff_transformer.py:320-336) and its kernel gathers
 * every feature row once per (row, neighbour, ic) (clustenwf_cuda_kernel.cu:41-47).
 * The order depends on nbhd_idx only; build it once per nbhd_idx and pass it as
 * row_order to clusten_wf_forward / clusten_wf_backward.  row_order may be NULL:
 * the rows are then taken in storage order (same results, more traffic).
 * n_out above 4096 is not handled (CLUSTEN_ERR_UNSUPPORTED): pass NULL then. */
CLUSTEN_API size_t clusten_wf_order_bytes(int b, int n_out);
CLUSTEN_API int clusten_wf_order_build(const int64_t* nbhd_idx, int b, int n_out, int m,
                                       void* row_order, size_t row_order_bytes, void* stream);

/* d_weights[b,i,j,ic] = sum_c feat[b,idx,c] * d_feat_new[b,i,ic,c]
 * d_feat[b,t,c] = sum_{(i,j): idx[b,i,j]==t} sum_ic d_feat_new[b,i,ic,c] * weights[b,i,j,ic]
 * replaces clusten_wf_backward (clustenwf_cuda.cpp:35-45, kernels :96-169).
 * inverse: built by clusten_inverse_build(nbhd_idx, b, n_out, m, n, ...). */
CLUSTEN_API int clusten_wf_backward(const void* d_feat_new, const void* weights, const void* feat,
                        const int64_t* nbhd_idx, const void* inverse, const void* row_order,
                        void* d_weights, void* d_feat,
                        int b, int n_out, int n, int m, int ic, int c, int dtype, void* stream);

/* ------------------------------------------------------------------------
 * Neighbourhood search on 2-D token positions: nn_idx[b,i,:] = the k database
 * points nearest to query[b,i] by Euclidean distance, ascending, ties towards
 * the lower index; nn_dist (may be NULL) receives the distances.
 * replaces knn_keops (models/point_utils.py:27-58; callers
 * models/aff_transformer.py:298 with k = 2 and :476 with k = 6), which the
 * reference evaluates with a pykeops LazyTensor argKmin.  fp32 positions
 * [b, n_query, 2] and [b, n, 2], int64 indices [b, n_query, k] like the
 * reference's.  Limits: k <= 8, k <= n, b <= 65535 (CLUSTEN_ERR_UNSUPPORTED).
 * ---------------------------------------------------------------------- */
CLUSTEN_API int clusten_knn2d(const float* query, const float* database, int b, int n_query, int n, int k,
                              int64_t* nn_idx, float* nn_dist, void* stream);

/* ------------------------------------------------------------------------
 * Neighbourhood tables of a stage in one pass: for token i, nearest cluster
 * r < nnc and member s < cs (slot j = r * cs + s), with
 * c = nearest_cluster[b,i,r] and t = member_idx[b,c,s]:
 *   nbhd_idx[b,i,j]  = t
 *   nbhd_mask[b,i,j] = cluster_mask[b,c,s]      (cluster_mask and nbhd_mask both given or both NULL)
 *   pe_idx[b,i,j]    = (int64)(rel.y * table_width + rel.x),
 *                      rel = pos[b,t] - (pos[b,i] - rel_pos_width), evaluated in fp32 in this order
 * replaces the three gathers and the elementwise arithmetic of BasicLayer.forward
 * (models/aff_transformer.py:476-487).  pos fp32 [b,n,2]; member_idx, cluster_mask
 * int64 [b,k,cs]; nearest_cluster int64 [b,n,nnc]; outputs int64 [b,n,nnc*cs].
 * A cluster id outside [0,k) gives nbhd_idx -1, mask 0 and pe_idx 0 for its cs
 * slots; a member outside [0,n) is passed through with pe_idx 0 (the reference's
 * gather is undefined for both).
 * ---------------------------------------------------------------------- */
CLUSTEN_API int clusten_nbhd_build(const float* pos, const int64_t* member_idx, const int64_t* cluster_mask,
                                   const int64_t* nearest_cluster, int64_t* nbhd_idx, int64_t* nbhd_mask,
                                   int64_t* pe_idx, int b, int n, int k, int cs, int nnc, int rel_pos_width,
                                   int table_width, void* stream);

/* ------------------------------------------------------------------------
 * Merge weights of ClusterMerging in one pass:
 *   weights[b,i,j,:] = weights_table[pe_idx[b,i,j],:] * (learned_prob[b, nbhd_idx[b,i,j]] * nbhd_mask[b,i,j])
 * replaces the table gather, the score gather and the elementwise products of
 * models/aff_transformer.py:340-358; the result is CLUSTENWF's first argument.
 * weights_table [table_rows, ic], learned_prob [b, n] (NULL = 1) and weights
 * [b, n_out, m, ic] share `dtype` (fp32 / fp16 / bf16); pe_idx, nbhd_idx and
 * nbhd_mask (NULL = 1) are int64 [b, n_out, m]; nbhd_idx is only read when
 * learned_prob is given.  A table row or a token out of range gives zero
 * weights (the reference's gathers are undefined there).
 * ---------------------------------------------------------------------- */
CLUSTEN_API int clusten_merge_weights(const void* weights_table, const int64_t* pe_idx, const void* learned_prob,
                                      const int64_t* nbhd_idx, const int64_t* nbhd_mask, void* weights, int b,
                                      int n_out, int n, int m, int ic, int table_rows, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CLUSTEN_B200_H_ */
