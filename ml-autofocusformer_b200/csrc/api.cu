// extern "C" entry points of libclusten_b200.so: argument checks and the
// choice between the tiled and the shape-agnostic kernels.  Declarations and
// the reference interfaces they replace are in include/clusten_b200.h.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"
#include "tiled.cuh"

namespace clusten {

static std::atomic<unsigned long long> g_launches{0};

void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

// ---- optional per-kernel timing -------------------------------------------------------------
namespace {
struct TimedLaunch {
    const char* name;
    cudaEvent_t start, stop;
};
std::atomic<int> g_timing{0};
std::mutex g_timing_mu;
std::vector<TimedLaunch> g_timed;
}  // namespace

ScopedKernelTimer::ScopedKernelTimer(const char* name, cudaStream_t s) : slot(-1), stream(s) {
    if (!g_timing.load(std::memory_order_relaxed)) return;
    TimedLaunch t{name, nullptr, nullptr};
    if (cudaEventCreate(&t.start) != cudaSuccess || cudaEventCreate(&t.stop) != cudaSuccess) {
        cudaGetLastError();
        return;
    }
    cudaEventRecord(t.start, s);
    std::lock_guard<std::mutex> lk(g_timing_mu);
    slot = (int)g_timed.size();
    g_timed.push_back(t);
}

ScopedKernelTimer::~ScopedKernelTimer() {
    if (slot < 0) return;
    std::lock_guard<std::mutex> lk(g_timing_mu);
    cudaEventRecord(g_timed[slot].stop, stream);
}

bool split_timing_labels() {
    static const bool on = [] {
        const char* v = getenv("CLUSTEN_SPLIT_TIMING");
        return v != nullptr && v[0] == '1';
    }();
    return on;
}

int check_launch() { return cudaGetLastError() == cudaSuccess ? CLUSTEN_OK : CLUSTEN_ERR_CUDA; }

int sm_count() {
    static std::mutex mu;
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lk(mu);
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

int resident_ctas(const void* kernel, int threads, size_t smem) {
    struct Key {
        const void* k; int dev; size_t smem; int threads;
        bool operator<(const Key& o) const {
            if (k != o.k) return k < o.k;
            if (dev != o.dev) return dev < o.dev;
            if (smem != o.smem) return smem < o.smem;
            return threads < o.threads;
        }
    };
    static std::mutex mu;
    static std::map<Key, int> cache;
    static std::map<std::pair<const void*, int>, size_t> limit;      // dynamic shared-memory limit set so far
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        cudaGetLastError();
        return CLUSTEN_ERR_CUDA;
    }
    const Key key{kernel, dev, smem, threads};
    std::lock_guard<std::mutex> lk(mu);
    // the limit is one number per kernel and device: it is only ever raised, so that a launch with a
    // smaller request does not take it away from a later launch with a larger one
    // (a kernel's static shared memory counts towards the 48 KB that need no opt-in, so the limit is raised well
    // before the dynamic part alone gets there)
    size_t& cur = limit[{kernel, dev}];
    if (smem > 32 * 1024 && smem > cur) {
        const size_t want = smem < 64 * 1024 ? 64 * 1024 : smem;
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)want) != cudaSuccess) {
            cudaGetLastError();
            return CLUSTEN_ERR_CUDA;
        }
        cur = want;
    }
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) != cudaSuccess) {
        cudaGetLastError();
        return CLUSTEN_ERR_CUDA;
    }
    if (per_sm < 1) per_sm = 1;
    cache[key] = per_sm;
    return per_sm;
}

namespace {

bool aligned(const void* p, size_t a) { return reinterpret_cast<uintptr_t>(p) % a == 0; }

// sizes common to QK and AV
int check_attn_args(int b, int h, int n, int m, int c, int dtype) {
    if (dtype_size(dtype) == 0) return CLUSTEN_ERR_DTYPE;
    if (b <= 0 || h <= 0 || n <= 0 || m <= 0 || c <= 0) return CLUSTEN_ERR_SHAPE;
    const long long lim = 0x7fffffffLL;
    if ((long long)b * h > lim || (long long)n * m > lim || (long long)n * c > lim) return CLUSTEN_ERR_SHAPE;
    return CLUSTEN_OK;
}

int check_wf_args(int b, int n_out, int n, int m, int ic, int c, int dtype) {
    if (dtype_size(dtype) == 0) return CLUSTEN_ERR_DTYPE;
    if (b <= 0 || n_out <= 0 || n <= 0 || m <= 0 || ic <= 0 || c <= 0) return CLUSTEN_ERR_SHAPE;
    const long long lim = 0x7fffffffLL;
    if ((long long)n_out * m * ic > lim || (long long)n * c > lim || (long long)n_out * ic * c > lim)
        return CLUSTEN_ERR_SHAPE;
    return CLUSTEN_OK;
}

int check_inverse_args(int b, int n_rows, int m, int nt) {
    if (b <= 0 || n_rows <= 0 || m <= 0 || nt <= 0) return CLUSTEN_ERR_SHAPE;
    if (m > 2048 || nt > kInvMaxTargets || (long long)n_rows * m >= 0x7fffffffLL) return CLUSTEN_ERR_UNSUPPORTED;
    return CLUSTEN_OK;
}

#define CLUSTEN_REQUIRE_PTR(p, a)                       \
    do {                                                \
        if ((p) == nullptr) return CLUSTEN_ERR_NULL;    \
        if (!aligned((p), (a))) return CLUSTEN_ERR_ALIGN; \
    } while (0)

}  // namespace

int validate_av_backward(const void* d_feat, const void* attn, const void* value, const int64_t* nbhd_idx,
                         const void* inverse, const void* d_attn, const void* d_value, int b, int h, int n, int m,
                         int c, int dtype) {
    int st = check_attn_args(b, h, n, m, c, dtype);
    if (st != CLUSTEN_OK) return st;
    st = check_inverse_args(b, n, m, n);
    if (st != CLUSTEN_OK) return st;
    const size_t es = dtype_size(dtype);
    CLUSTEN_REQUIRE_PTR(d_feat, es);
    CLUSTEN_REQUIRE_PTR(attn, es);
    CLUSTEN_REQUIRE_PTR(value, es);
    CLUSTEN_REQUIRE_PTR(nbhd_idx, 8);
    CLUSTEN_REQUIRE_PTR(inverse, 16);
    CLUSTEN_REQUIRE_PTR(d_attn, es);
    CLUSTEN_REQUIRE_PTR(d_value, es);
    return CLUSTEN_OK;
}

}  // namespace clusten

using namespace clusten;

extern "C" {

const char* clusten_status_string(int status) {
    switch (status) {
        case CLUSTEN_OK: return "CLUSTEN_OK";
        case CLUSTEN_ERR_DTYPE: return "CLUSTEN_ERR_DTYPE: unknown element type";
        case CLUSTEN_ERR_SHAPE: return "CLUSTEN_ERR_SHAPE: a size is not positive or too large";
        case CLUSTEN_ERR_NULL: return "CLUSTEN_ERR_NULL: a required pointer is NULL";
        case CLUSTEN_ERR_ALIGN: return "CLUSTEN_ERR_ALIGN: a pointer is not aligned to its element size";
        case CLUSTEN_ERR_WORKSPACE: return "CLUSTEN_ERR_WORKSPACE: inverse-index buffer too small";
        case CLUSTEN_ERR_UNSUPPORTED: return "CLUSTEN_ERR_UNSUPPORTED: size outside the supported range";
        case CLUSTEN_ERR_CUDA: return "CLUSTEN_ERR_CUDA: the CUDA runtime reported an error";
        case CLUSTEN_ERR_NOALLOC_CAPACITY:
            return "CLUSTEN_ERR_NOALLOC_CAPACITY: sizes exceed the built-in inverse-index array of "
                   "clusten_av_backward_noalloc (CLUSTEN_NOALLOC_MAX_INTS)";
        default: return "CLUSTEN: unknown status";
    }
}

int clusten_version(void) { return 100; }

int clusten_timing_enable(int on) {
    g_timing.store(on ? 1 : 0, std::memory_order_relaxed);
    return CLUSTEN_OK;
}

int clusten_timing_collect(char* buf, size_t buf_bytes) {
    if (buf == nullptr || buf_bytes == 0) return CLUSTEN_ERR_NULL;
    std::vector<TimedLaunch> taken;
    {
        std::lock_guard<std::mutex> lk(g_timing_mu);
        taken.swap(g_timed);
    }
    std::map<std::string, std::pair<long long, double>> acc;
    std::vector<std::string> order;
    int status = CLUSTEN_OK;
    for (auto& t : taken) {
        float ms = 0.f;
        if (cudaEventSynchronize(t.stop) != cudaSuccess || cudaEventElapsedTime(&ms, t.start, t.stop) != cudaSuccess) {
            cudaGetLastError();
            status = CLUSTEN_ERR_CUDA;
        } else {
            auto it = acc.find(t.name);
            if (it == acc.end()) {
                order.push_back(t.name);
                acc[t.name] = {1, ms};
            } else {
                it->second.first += 1;
                it->second.second += ms;
            }
        }
        cudaEventDestroy(t.start);
        cudaEventDestroy(t.stop);
    }
    if (status != CLUSTEN_OK) return status;
    std::string out;
    char line[256];
    for (auto& name : order) {
        snprintf(line, sizeof line, "%s %lld %.6f\n", name.c_str(), acc[name].first, acc[name].second);
        out += line;
    }
    const size_t n = out.size() < buf_bytes - 1 ? out.size() : buf_bytes - 1;
    memcpy(buf, out.data(), n);
    buf[n] = 0;
    return (int)order.size();
}

unsigned long long clusten_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

size_t clusten_inverse_bytes(int b, int n_rows, int m, int n_targets) {
    if (check_inverse_args(b, n_rows, m, n_targets) != CLUSTEN_OK) return 0;
    return inverse_ints(b, n_rows, m, n_targets) * sizeof(int);
}

int clusten_inverse_build(const int64_t* nbhd_idx, int b, int n_rows, int m, int n_targets, void* inverse,
                          size_t inverse_bytes, void* stream) {
    const int st = check_inverse_args(b, n_rows, m, n_targets);
    if (st != CLUSTEN_OK) return st;
    CLUSTEN_REQUIRE_PTR(nbhd_idx, 8);
    CLUSTEN_REQUIRE_PTR(inverse, 16);
    if (inverse_bytes < inverse_ints(b, n_rows, m, n_targets) * sizeof(int)) return CLUSTEN_ERR_WORKSPACE;
    return launch_inverse_build(nbhd_idx, b, n_rows, m, n_targets, inverse, (cudaStream_t)stream);
}

int clusten_qk_forward(const void* query, const void* key, const int64_t* nbhd_idx, void* attn, int b, int h,
                       int n, int m, int c, int dtype, void* stream) {
    const int st = check_attn_args(b, h, n, m, c, dtype);
    if (st != CLUSTEN_OK) return st;
    const size_t es = dtype_size(dtype);
    CLUSTEN_REQUIRE_PTR(query, es);
    CLUSTEN_REQUIRE_PTR(key, es);
    CLUSTEN_REQUIRE_PTR(nbhd_idx, 8);
    CLUSTEN_REQUIRE_PTR(attn, es);
    cudaStream_t s = (cudaStream_t)stream;
    if (tiled_dot_supported(dtype, query, key, attn, n, m, c))
        return launch_tiled_dot("qk_forward", dtype, key, query, nbhd_idx, attn, b, h, n, m, s);
    return launch_gather_dot("qk_forward", dtype, key, query, nbhd_idx, attn, b * h, h, n, n, m, 1, c, s);
}

// element strides (batch, head, row) of a [b, h, n, c] view with contiguous rows -> usable by the tiled kernels?
static bool view_ok(const void* p, const long long* st, int esize) {
    if (!aligned(p, 16)) return false;
    for (int i = 0; i < 3; ++i)
        if (st[i] < 0 || (st[i] * esize) % 16 != 0) return false;
    return st[2] > 0 && st[2] <= (1ll << 30);            // the kernels keep the row stride in 32 bits
}

int clusten_qk_forward_strided(const void* query, const long long* query_strides, const void* key,
                               const long long* key_strides, const int64_t* nbhd_idx, void* attn, int b, int h, int n,
                               int m, int c, int dtype, void* stream) {
    const int st = check_attn_args(b, h, n, m, c, dtype);
    if (st != CLUSTEN_OK) return st;
    const size_t es = dtype_size(dtype);
    CLUSTEN_REQUIRE_PTR(query, es);
    CLUSTEN_REQUIRE_PTR(key, es);
    CLUSTEN_REQUIRE_PTR(nbhd_idx, 8);
    CLUSTEN_REQUIRE_PTR(attn, es);
    if (query_strides == nullptr || key_strides == nullptr) return CLUSTEN_ERR_NULL;
    if (!tiled_dot_supported(dtype, query, key, attn, n, m, c) || !view_ok(query, query_strides, (int)es) ||
        !view_ok(key, key_strides, (int)es))
        return CLUSTEN_ERR_UNSUPPORTED;
    GatherStrides gs{};
    gs.x_batch = key_strides[0];  gs.x_head = key_strides[1];  gs.x_row = key_strides[2];
    gs.y_batch = query_strides[0];  gs.y_head = query_strides[1];  gs.y_row = query_strides[2];
    return launch_tiled_dot("qk_forward", dtype, key, query, nbhd_idx, attn, b, h, n, m, (cudaStream_t)stream, gs);
}

int clusten_av_forward_strided(const void* attn, const void* value, const long long* value_strides,
                               const int64_t* nbhd_idx, void* feat, int b, int h, int n, int m, int c, int dtype,
                               void* stream) {
    const int st = check_attn_args(b, h, n, m, c, dtype);
    if (st != CLUSTEN_OK) return st;
    const size_t es = dtype_size(dtype);
    CLUSTEN_REQUIRE_PTR(attn, es);
    CLUSTEN_REQUIRE_PTR(value, es);
    CLUSTEN_REQUIRE_PTR(nbhd_idx, 8);
    CLUSTEN_REQUIRE_PTR(feat, es);
    if (value_strides == nullptr) return CLUSTEN_ERR_NULL;
    if (!tiled_sum_supported(dtype, attn, value, feat, n, m, c) || !view_ok(value, value_strides, (int)es))
        return CLUSTEN_ERR_UNSUPPORTED;
    GatherStrides gs{};
    gs.x_batch = value_strides[0];  gs.x_head = value_strides[1];  gs.x_row = value_strides[2];
    return launch_tiled_sum("av_forward", dtype, attn, value, nbhd_idx, feat, b, h, n, m, (cudaStream_t)stream, gs);
}

int clusten_local_attention_forward(const void* query, const long long* query_strides, const void* key,
                                    const void* value, const long long* kv_strides, const int64_t* nbhd_idx,
                                    const void* pos_bias, const void* pe_table, const int64_t* pe_idx, int table_rows,
                                    const int64_t* mask, const void* blank_k, const void* blank_v, void* out, int b,
                                    int h, int n, int m, int c, int dtype, void* stream) {
    const int st = check_attn_args(b, h, n, m, c, dtype);
    if (st != CLUSTEN_OK) return st;
    const int es = dtype_size(dtype);
    CLUSTEN_REQUIRE_PTR(query, 16);
    CLUSTEN_REQUIRE_PTR(key, 16);
    CLUSTEN_REQUIRE_PTR(value, 16);
    CLUSTEN_REQUIRE_PTR(nbhd_idx, 8);
    CLUSTEN_REQUIRE_PTR(out, 16);
    if (pos_bias && !aligned(pos_bias, es)) return CLUSTEN_ERR_ALIGN;
    if ((pe_table == nullptr) != (pe_idx == nullptr)) return CLUSTEN_ERR_NULL;
    if (pe_table && (!aligned(pe_table, es) || !aligned(pe_idx, 8) || table_rows <= 0)) return CLUSTEN_ERR_ALIGN;
    if (mask && !aligned(mask, 8)) return CLUSTEN_ERR_ALIGN;
    if ((blank_k == nullptr) != (blank_v == nullptr)) return CLUSTEN_ERR_NULL;
    if (blank_k && (!aligned(blank_k, 16) || !aligned(blank_v, 16))) return CLUSTEN_ERR_ALIGN;
    if (!fused_attention_supported(dtype, n, m, c)) return CLUSTEN_ERR_UNSUPPORTED;
    GatherStrides gs{};
    if (query_strides) {
        if (!view_ok(query, query_strides, es)) return CLUSTEN_ERR_UNSUPPORTED;
        gs.y_batch = query_strides[0];  gs.y_head = query_strides[1];  gs.y_row = query_strides[2];
    }
    if (kv_strides) {
        if (!view_ok(key, kv_strides, es) || !view_ok(value, kv_strides, es)) return CLUSTEN_ERR_UNSUPPORTED;
        gs.x_batch = kv_strides[0];  gs.x_head = kv_strides[1];  gs.x_row = kv_strides[2];
    }
    return launch_fused_attention(dtype, query, key, value, nbhd_idx, pos_bias, pe_table, pe_idx, table_rows, mask,
                                  blank_k, blank_v, out, b, h, n, m, gs, (cudaStream_t)stream);
}

int clusten_qk_backward(const void* d_attn, const void* query, const void* key, const int64_t* nbhd_idx,
                        const void* inverse, void* d_query, void* d_key, int b, int h, int n, int m, int c,
                        int dtype, void* stream) {
    int st = check_attn_args(b, h, n, m, c, dtype);
    if (st != CLUSTEN_OK) return st;
    st = check_inverse_args(b, n, m, n);
    if (st != CLUSTEN_OK) return st;
    const size_t es = dtype_size(dtype);
    CLUSTEN_REQUIRE_PTR(d_attn, es);
    CLUSTEN_REQUIRE_PTR(query, es);
    CLUSTEN_REQUIRE_PTR(key, es);
    CLUSTEN_REQUIRE_PTR(nbhd_idx, 8);
    CLUSTEN_REQUIRE_PTR(inverse, 16);
    CLUSTEN_REQUIRE_PTR(d_query, es);
    CLUSTEN_REQUIRE_PTR(d_key, es);
    cudaStream_t s = (cudaStream_t)stream;
    const InverseView inv = inverse_view(inverse, b, n, m, n);
    // d_query: weighted sum of gathered keys
    if (tiled_sum_supported(dtype, d_attn, key, d_query, n, m, c))
        st = launch_tiled_sum("qk_d_query", dtype, d_attn, key, nbhd_idx, d_query, b, h, n, m, s);
    else
        st = launch_gather_sum("qk_d_query", dtype, d_attn, key, nbhd_idx, d_query, b * h, h, n, n, m, 1, c, s);
    if (st != CLUSTEN_OK) return st;
    // d_key: segmented reduction of d_attn * query over the inverse index
    if (tiled_scatter_supported(dtype, d_attn, query, d_key, n, m, c))
        return launch_tiled_scatter("qk_d_key", dtype, d_attn, query, nbhd_idx, inv, d_key, b, h, n, m, s);
    return launch_scatter_sum("qk_d_key", dtype, d_attn, query, nbhd_idx, inv, d_key, b * h, h, n, n, m, 1, c, s);
}

int clusten_av_forward(const void* attn, const void* value, const int64_t* nbhd_idx, void* feat, int b, int h,
                       int n, int m, int c, int dtype, void* stream) {
    const int st = check_attn_args(b, h, n, m, c, dtype);
    if (st != CLUSTEN_OK) return st;
    const size_t es = dtype_size(dtype);
    CLUSTEN_REQUIRE_PTR(attn, es);
    CLUSTEN_REQUIRE_PTR(value, es);
    CLUSTEN_REQUIRE_PTR(nbhd_idx, 8);
    CLUSTEN_REQUIRE_PTR(feat, es);
    cudaStream_t s = (cudaStream_t)stream;
    if (tiled_sum_supported(dtype, attn, value, feat, n, m, c))
        return launch_tiled_sum("av_forward", dtype, attn, value, nbhd_idx, feat, b, h, n, m, s);
    return launch_gather_sum("av_forward", dtype, attn, value, nbhd_idx, feat, b * h, h, n, n, m, 1, c, s);
}

int clusten_av_backward(const void* d_feat, const void* attn, const void* value, const int64_t* nbhd_idx,
                        const void* inverse, void* d_attn, void* d_value, int b, int h, int n, int m, int c,
                        int dtype, void* stream) {
    int st = validate_av_backward(d_feat, attn, value, nbhd_idx, inverse, d_attn, d_value, b, h, n, m, c, dtype);
    if (st != CLUSTEN_OK) return st;
    cudaStream_t s = (cudaStream_t)stream;
    const InverseView inv = inverse_view(inverse, b, n, m, n);
    // d_attn: dot of each gathered value row with the row's d_feat
    if (tiled_dot_supported(dtype, d_feat, value, d_attn, n, m, c))
        st = launch_tiled_dot("av_d_attn", dtype, value, d_feat, nbhd_idx, d_attn, b, h, n, m, s);
    else
        st = launch_gather_dot("av_d_attn", dtype, value, d_feat, nbhd_idx, d_attn, b * h, h, n, n, m, 1, c, s);
    if (st != CLUSTEN_OK) return st;
    // d_value: segmented reduction of attn * d_feat over the inverse index
    if (tiled_scatter_supported(dtype, attn, d_feat, d_value, n, m, c))
        return launch_tiled_scatter("av_d_value", dtype, attn, d_feat, nbhd_idx, inv, d_value, b, h, n, m, s);
    return launch_scatter_sum("av_d_value", dtype, attn, d_feat, nbhd_idx, inv, d_value, b * h, h, n, n, m, 1, c, s);
}

int clusten_knn2d(const float* query, const float* database, int b, int n_query, int n, int k, int64_t* nn_idx,
                  float* nn_dist, void* stream) {
    if (b <= 0 || n_query <= 0 || n <= 0 || k <= 0) return CLUSTEN_ERR_SHAPE;
    if (k > 8 || k > n || b > 65535) return CLUSTEN_ERR_UNSUPPORTED;
    CLUSTEN_REQUIRE_PTR(query, 8);
    CLUSTEN_REQUIRE_PTR(database, 8);
    CLUSTEN_REQUIRE_PTR(nn_idx, 8);
    if (nn_dist && !aligned(nn_dist, 4)) return CLUSTEN_ERR_ALIGN;
    return launch_knn2d(query, database, b, n_query, n, k, nn_idx, nn_dist, (cudaStream_t)stream);
}

int clusten_nbhd_build(const float* pos, const int64_t* member_idx, const int64_t* cluster_mask,
                       const int64_t* nearest_cluster, int64_t* nbhd_idx, int64_t* nbhd_mask, int64_t* pe_idx, int b,
                       int n, int k, int cs, int nnc, int rel_pos_width, int table_width, void* stream) {
    if (b <= 0 || n <= 0 || k <= 0 || cs <= 0 || nnc <= 0 || table_width <= 0) return CLUSTEN_ERR_SHAPE;
    if ((long long)nnc * cs > 0x7fffffffLL || (long long)b * n > 0x7fffffffLL) return CLUSTEN_ERR_SHAPE;
    CLUSTEN_REQUIRE_PTR(pos, 8);
    CLUSTEN_REQUIRE_PTR(member_idx, 8);
    CLUSTEN_REQUIRE_PTR(nearest_cluster, 8);
    CLUSTEN_REQUIRE_PTR(nbhd_idx, 8);
    CLUSTEN_REQUIRE_PTR(pe_idx, 8);
    if ((cluster_mask == nullptr) != (nbhd_mask == nullptr)) return CLUSTEN_ERR_NULL;
    if (cluster_mask && (!aligned(cluster_mask, 8) || !aligned(nbhd_mask, 8))) return CLUSTEN_ERR_ALIGN;
    return launch_nbhd_build(pos, member_idx, cluster_mask, nearest_cluster, nbhd_idx, nbhd_mask, pe_idx, b, n, k, cs,
                             nnc, rel_pos_width, table_width, (cudaStream_t)stream);
}

int clusten_merge_weights(const void* weights_table, const int64_t* pe_idx, const void* learned_prob,
                          const int64_t* nbhd_idx, const int64_t* nbhd_mask, void* weights, int b, int n_out, int n,
                          int m, int ic, int table_rows, int dtype, void* stream) {
    if (b <= 0 || n_out <= 0 || n <= 0 || m <= 0 || ic <= 0 || table_rows <= 0) return CLUSTEN_ERR_SHAPE;
    if ((long long)b * n > 0x7fffffffLL || (long long)table_rows * ic > 0x7fffffffLL) return CLUSTEN_ERR_SHAPE;
    if (dtype != CLUSTEN_F32 && dtype != CLUSTEN_F16 && dtype != CLUSTEN_BF16) return CLUSTEN_ERR_DTYPE;
    const size_t es = dtype_size(dtype);
    CLUSTEN_REQUIRE_PTR(weights_table, es);
    CLUSTEN_REQUIRE_PTR(pe_idx, 8);
    CLUSTEN_REQUIRE_PTR(weights, es);
    if (learned_prob) {
        if (!aligned(learned_prob, es)) return CLUSTEN_ERR_ALIGN;
        CLUSTEN_REQUIRE_PTR(nbhd_idx, 8);
    }
    if (nbhd_mask && !aligned(nbhd_mask, 8)) return CLUSTEN_ERR_ALIGN;
    return launch_merge_weights(dtype, weights_table, pe_idx, learned_prob, nbhd_idx, nbhd_mask, weights, b, n_out, n,
                                m, ic, table_rows, (cudaStream_t)stream);
}

size_t clusten_wf_order_bytes(int b, int n_out) {
    if (b < 1 || n_out < 1) return 0;
    return wf_order_bytes(b, n_out);
}

int clusten_wf_order_build(const int64_t* nbhd_idx, int b, int n_out, int m, void* row_order, size_t row_order_bytes,
                           void* stream) {
    if (b < 1 || n_out < 1 || m < 1) return CLUSTEN_ERR_SHAPE;
    CLUSTEN_REQUIRE_PTR(nbhd_idx, 8);
    CLUSTEN_REQUIRE_PTR(row_order, 4);
    if (row_order_bytes < wf_order_bytes(b, n_out)) return CLUSTEN_ERR_WORKSPACE;
    return launch_wf_order(nbhd_idx, b, n_out, m, static_cast<int*>(row_order), (cudaStream_t)stream);
}

int clusten_wf_forward(const void* weights, const void* feat, const int64_t* nbhd_idx, const void* row_order,
                       void* feat_new, int b, int n_out, int n, int m, int ic, int c, int dtype, void* stream) {
    const int st = check_wf_args(b, n_out, n, m, ic, c, dtype);
    if (st != CLUSTEN_OK) return st;
    const size_t es = dtype_size(dtype);
    CLUSTEN_REQUIRE_PTR(weights, es);
    CLUSTEN_REQUIRE_PTR(feat, es);
    CLUSTEN_REQUIRE_PTR(nbhd_idx, 8);
    CLUSTEN_REQUIRE_PTR(feat_new, es);
    if (row_order && reinterpret_cast<uintptr_t>(row_order) % 4 != 0) return CLUSTEN_ERR_ALIGN;
    if (tiled_wf_gather_supported(dtype, weights, feat, feat_new, n_out, n, m, ic, c))
        return launch_tiled_wf_sum("wf_forward", dtype, weights, feat, nbhd_idx, static_cast<const int*>(row_order),
                                   feat_new, b, n_out, n, m, ic, c, (cudaStream_t)stream);
    return launch_gather_sum("wf_forward", dtype, weights, feat, nbhd_idx, feat_new, b, 1, n_out, n, m, ic, c,
                             (cudaStream_t)stream);
}

int clusten_wf_backward(const void* d_feat_new, const void* weights, const void* feat, const int64_t* nbhd_idx,
                        const void* inverse, const void* row_order, void* d_weights, void* d_feat, int b, int n_out,
                        int n, int m, int ic, int c, int dtype, void* stream) {
    int st = check_wf_args(b, n_out, n, m, ic, c, dtype);
    if (st != CLUSTEN_OK) return st;
    st = check_inverse_args(b, n_out, m, n);
    if (st != CLUSTEN_OK) return st;
    const size_t es = dtype_size(dtype);
    CLUSTEN_REQUIRE_PTR(d_feat_new, es);
    CLUSTEN_REQUIRE_PTR(weights, es);
    CLUSTEN_REQUIRE_PTR(feat, es);
    CLUSTEN_REQUIRE_PTR(nbhd_idx, 8);
    CLUSTEN_REQUIRE_PTR(inverse, 16);
    CLUSTEN_REQUIRE_PTR(d_weights, es);
    CLUSTEN_REQUIRE_PTR(d_feat, es);
    cudaStream_t s = (cudaStream_t)stream;
    const InverseView inv = inverse_view(inverse, b, n_out, m, n);
    if (row_order && reinterpret_cast<uintptr_t>(row_order) % 4 != 0) return CLUSTEN_ERR_ALIGN;
    if (tiled_wf_gather_supported(dtype, d_weights, feat, d_feat_new, n_out, n, m, ic, c))
        st = launch_tiled_wf_dot("wf_d_weights", dtype, feat, d_feat_new, nbhd_idx, static_cast<const int*>(row_order),
                                 d_weights, b, n_out, n, m, ic, c, s);
    else
        st = launch_gather_dot("wf_d_weights", dtype, feat, d_feat_new, nbhd_idx, d_weights, b, 1, n_out, n, m, ic, c, s);
    if (st != CLUSTEN_OK) return st;
    if (tiled_wf_dfeat_supported(dtype, weights, d_feat_new, d_feat, n_out, n, m, ic, c))
        return launch_tiled_wf_dfeat("wf_d_feat", dtype, weights, d_feat_new, nbhd_idx, inv, d_feat, b, n_out, n, m, ic,
                                     c, s);
    if (tiled_wf_scatter_supported(dtype, weights, d_feat_new, d_feat, n_out, n, m, ic, c))
        return launch_tiled_wf_scatter("wf_d_feat", dtype, weights, d_feat_new, nbhd_idx, inv, d_feat, b, n_out, n, m,
                                       ic, c, s);
    return launch_scatter_sum("wf_d_feat", dtype, weights, d_feat_new, nbhd_idx, inv, d_feat, b, 1, n_out, n, m, ic, c, s);
}

}  // extern "C"
