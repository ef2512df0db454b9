// clusten_av_backward_noalloc: CLUSTENAV backward for callers that cannot obtain device memory at
// call time.
//
// The scatter-side gradient needs the inverse neighbour index, which the regular entry point
// (clusten_av_backward) takes as a caller-provided buffer.  Some hosts have no buffer to give: an
// inference engine's enqueue callback, or any program that hands all device memory to its own pool
// up front, may neither call cudaMalloc (it can fail, and it synchronises the device) nor ask the
// pool from inside the callback.  For them the inverse index lives in the fixed array below, which
// every GPU that loads this library holds until the process exits (kStaticInverseInts * 4 bytes,
// about 13.6 MB).  Nothing here allocates: no cudaMalloc / cudaFree and no allocating library call.
//
// In host code `g_static_inverse` is only a stand-in for the device array, never a device address;
// the address a kernel may use comes from cudaGetSymbolAddress, taken once per device, with that
// device current, the first time the entry point runs there (that first call therefore does a little
// set-up work and should come before any stream capture).  All calls share the one array: it keeps
// the previous call's contents, the build re-initialises everything it later reads, and two calls
// that overlap on the GPU (different streams or threads) race on it.  The looked-up address is kept
// per device ordinal for the life of the process; it belongs to the device's primary context, so a
// program that calls cudaDeviceReset must not use this entry point afterwards.
#include <mutex>

#include "common.cuh"
#include "tiled.cuh"

namespace clusten {

namespace {

static __device__ __align__(256) int g_static_inverse[CLUSTEN_NOALLOC_MAX_INTS];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mu;
int* g_static_ptr[kMaxDevices] = {nullptr};

// device address of g_static_inverse on the current device; nullptr on failure
int* static_inverse_address() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        cudaGetLastError();
        return nullptr;
    }
    std::lock_guard<std::mutex> lk(g_setup_mu);
    if (g_static_ptr[dev] == nullptr) {
        int* ptr = nullptr;
        if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_inverse) != cudaSuccess || ptr == nullptr) {
            cudaGetLastError();
            return nullptr;
        }
        g_static_ptr[dev] = ptr;
    }
    return g_static_ptr[dev];
}

}  // namespace
}  // namespace clusten

using namespace clusten;

extern "C" int clusten_av_backward_noalloc(const void* d_feat, const void* attn, const void* value,
                                           const int64_t* nbhd_idx, void* d_attn, void* d_value, int b, int h,
                                           int n, int m, int c, int dtype, void* stream) {
    if (dtype_size(dtype) == 0) return CLUSTEN_ERR_DTYPE;
    if (b <= 0 || h <= 0 || n <= 0 || m <= 0 || c <= 0) return CLUSTEN_ERR_SHAPE;
    if (clusten_inverse_bytes(b, n, m, n) == 0) return CLUSTEN_ERR_UNSUPPORTED;
    // the fixed array must hold the whole inverse index of this call
    if (inverse_ints(b, n, m, n) > (size_t)CLUSTEN_NOALLOC_MAX_INTS) return CLUSTEN_ERR_NOALLOC_CAPACITY;
    int* inverse = static_inverse_address();
    if (inverse == nullptr) return CLUSTEN_ERR_CUDA;
    // every check of the regular entry point runs before anything is launched, so a rejected call
    // neither touches the shared array nor spends a launch
    int st = validate_av_backward(d_feat, attn, value, nbhd_idx, inverse, d_attn, d_value, b, h, n, m, c, dtype);
    if (st != CLUSTEN_OK) return st;
    st = clusten_inverse_build(nbhd_idx, b, n, m, n, inverse, (size_t)CLUSTEN_NOALLOC_MAX_INTS * sizeof(int),
                                   stream);
    if (st != CLUSTEN_OK) return st;
    return clusten_av_backward(d_feat, attn, value, nbhd_idx, inverse, d_attn, d_value, b, h, n, m, c, dtype,
                               stream);
}
