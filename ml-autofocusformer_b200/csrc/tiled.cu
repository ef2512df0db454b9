#include "tiled.cuh"

namespace clusten {

bool tiled_sum_supported(int, const void*, const void*, const void*, int, int, int) { return false; }
int launch_tiled_sum(int, const void*, const void*, const int64_t*, void*, int, int, int, int, cudaStream_t) {
    return CLUSTEN_ERR_UNSUPPORTED;
}
bool tiled_dot_supported(int, const void*, const void*, const void*, int, int, int) { return false; }
int launch_tiled_dot(int, const void*, const void*, const int64_t*, void*, int, int, int, int, cudaStream_t) {
    return CLUSTEN_ERR_UNSUPPORTED;
}
bool tiled_scatter_supported(int, const void*, const void*, const void*, int, int, int) { return false; }
int launch_tiled_scatter(int, const void*, const void*, const int64_t*, const InverseView&, void*, int, int, int,
                         int, cudaStream_t) {
    return CLUSTEN_ERR_UNSUPPORTED;
}

}  // namespace clusten
