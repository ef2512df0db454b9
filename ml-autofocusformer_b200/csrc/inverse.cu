// Inverse neighbour index: for every target token the list of (row, slot)
// pairs of nbhd_idx that point at it, ordered by row.  It turns the
// reference's atomicAdd scatter for d_key / d_value / d_feat
// (clusten/src/clustenqk_cuda_kernel.cu:125, clustenav_cuda_kernel.cu:121,
// clustenwf_cuda_kernel.cu:129) into a gather with a fixed summation order.
//
// One CTA per batch element.  Counters live in shared memory; the only
// atomics are integer adds and ORs, whose results do not depend on the order
// in which they are applied, so the buffer contents are deterministic.
#include "common.cuh"

namespace clusten {

namespace {

constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;

// P > 0: number of 32-slot passes over a row (m <= 32 P), rows kept in registers; P == 0: any m.
template <int P>
__global__ void __launch_bounds__(kThreads)
inverse_build_kernel(const int64_t* __restrict__ idx, int n_rows, int m, int nt, int* __restrict__ header,
                     int* __restrict__ rowptr, int* __restrict__ seglen, int* __restrict__ entries,
                     int* __restrict__ scratch, int* __restrict__ tileflag, int ntiles) {
    extern __shared__ int sm[];
    // the three per-target arrays: in shared memory, or (more targets than fit there) in this batch
    // element's part of the global scratch; the block barriers below order the accesses either way
    int* counters = scratch ? scratch + (long long)blockIdx.x * 3 * nt : sm;
    int* base = counters;                                              // running write position of target t
    unsigned* mask = reinterpret_cast<unsigned*>(counters + nt);       // rows of the current group that hit t
    unsigned* dupm = reinterpret_cast<unsigned*>(counters + 2 * nt);   // rows that hit t more than once
    __shared__ int warp_tot[kWarps];

    const int b = blockIdx.x;
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const long long E = (long long)n_rows * m;
    const int64_t* ib = idx + (long long)b * E;
    int* rp = rowptr + (long long)b * (nt + 1);
    int* ent = entries + (long long)b * E;

    if (b == 0 && tid == 0) {
        header[0] = (int)kInvMagic;
        header[1] = gridDim.x;
        header[2] = n_rows;
        header[3] = m;
        header[4] = nt;
    }
    {   // batch elements the structured build has done are skipped; the others have no structured tile
        int* tf = tileflag + (long long)b * (1 + ntiles);
        if (tf[0] != kBuildGeneral) return;
        for (int t = tid; t < ntiles; t += kThreads) tf[1 + t] = kTileGeneral;
    }
    for (int t = tid; t < nt; t += kThreads) {
        base[t] = 0;
        mask[t] = 0u;
        dupm[t] = 0u;
    }
    __syncthreads();

    // pass 1: how often each target is referenced (upper bound of its segment length)
    int oob = 0;
    for (long long e = tid; e < E; e += kThreads) {
        const long long tk = ib[e];
        if (tk >= 0 && tk < nt) atomicAdd(&base[(int)tk], 1);
        else ++oob;
    }
    if (oob) atomicAdd(&header[5], oob);
    __syncthreads();

    // exclusive scan of the counts -> segment starts
    {
        const int per = (nt + kThreads - 1) / kThreads;
        const int lo = min(tid * per, nt);
        const int hi = min(lo + per, nt);
        int local = 0;
        for (int t = lo; t < hi; ++t) local += base[t];
        int incl = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int y = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += y;
        }
        if (lane == 31) warp_tot[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int w = warp_tot[lane];
            int wi = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int y = __shfl_up_sync(0xffffffffu, wi, o);
                if (lane >= o) wi += y;
            }
            warp_tot[lane] = wi - w;   // exclusive
        }
        __syncthreads();
        int run = warp_tot[warp] + incl - local;
        for (int t = lo; t < hi; ++t) {
            const int cnt = base[t];
            base[t] = run;
            rp[t] = run;
            run += cnt;
        }
        if (hi == nt && lo < nt) rp[nt] = run;
        if (nt == 0 && tid == 0) rp[0] = 0;
    }
    __syncthreads();

    // pass 2: 32 rows at a time, one warp per row.  Within a group the position of
    // row r inside target t's segment is the number of lower rows of the group that
    // also hit t, read off a 32-bit row mask.
    const unsigned bit = 1u << warp;
    if (P > 0) {
        // m <= 32 P: a lane keeps its P slots of the row in registers; the next group's slots are
        // loaded before the current group is processed
        int cur[P > 0 ? P : 1], nxt[P > 0 ? P : 1];
        auto load_row = [&](int row, int (&dst)[P > 0 ? P : 1]) {
#pragma unroll
            for (int p = 0; p < P; ++p) {
                const int j = lane + 32 * p;
                long long tk = -1;
                if (row < n_rows && j < m) tk = ib[(long long)row * m + j];
                dst[p] = (tk >= 0 && tk < nt) ? (int)tk : -1;
            }
        };
        load_row(warp, cur);
        for (int g0 = 0; g0 < n_rows; g0 += kWarps) {
            const int row = g0 + warp;
            load_row(row + kWarps, nxt);
            unsigned win = 0u, last = 0u;
#pragma unroll
            for (int p = 0; p < P; ++p) {
                if (cur[p] >= 0) {
                    const unsigned old = atomicOr(&mask[cur[p]], bit);
                    if (old & bit) atomicOr(&dupm[cur[p]], bit);
                    else win |= 1u << p;
                }
            }
            __syncthreads();
#pragma unroll
            for (int p = 0; p < P; ++p) {
                if ((win >> p) & 1u) {
                    const int tk = cur[p];
                    const unsigned mk = mask[tk];
                    const int pos = base[tk] + __popc(mk & (bit - 1u));
                    const bool dup = (dupm[tk] & bit) != 0u;
                    ent[pos] = dup ? (int)(kDupFlag | (unsigned)(row * m)) : (row * m + lane + 32 * p);
                    if ((mk >> warp) == 1u) last |= 1u << p;
                }
            }
            __syncthreads();
#pragma unroll
            for (int p = 0; p < P; ++p) {
                if ((last >> p) & 1u) {
                    const int tk = cur[p];
                    base[tk] += __popc(mask[tk]);
                    mask[tk] = 0u;
                    dupm[tk] = 0u;
                }
            }
            __syncthreads();
#pragma unroll
            for (int p = 0; p < P; ++p) cur[p] = nxt[p];
        }
    } else {
    for (int g0 = 0; g0 < n_rows; g0 += kWarps) {
        const int row = g0 + warp;
        const bool live = row < n_rows;
        const int64_t* irow = ib + (long long)row * m;
        unsigned long long win = 0ull, last = 0ull;   // per 32-slot pass: this lane placed the entry / closes the group
        if (live) {
            for (int p = 0, j = lane; j < m; ++p, j += 32) {
                const long long tk = irow[j];
                if (tk >= 0 && tk < nt) {
                    const unsigned old = atomicOr(&mask[(int)tk], bit);
                    if (old & bit) atomicOr(&dupm[(int)tk], bit);
                    else win |= 1ull << p;
                }
            }
        }
        __syncthreads();
        if (live) {
            for (int p = 0, j = lane; j < m; ++p, j += 32) {
                if (!((win >> p) & 1ull)) continue;
                const int tk = (int)irow[j];
                const unsigned mk = mask[tk];
                const int pos = base[tk] + __popc(mk & (bit - 1u));
                const bool dup = (dupm[tk] & bit) != 0u;
                ent[pos] = dup ? (int)(kDupFlag | (unsigned)(row * m)) : (row * m + j);
                if ((mk >> warp) == 1u) last |= 1ull << p;
            }
        }
        __syncthreads();
        if (live) {
            for (int p = 0, j = lane; j < m; ++p, j += 32) {
                if (!((last >> p) & 1ull)) continue;
                const int tk = (int)irow[j];
                base[tk] += __popc(mask[tk]);
                mask[tk] = 0u;
                dupm[tk] = 0u;
            }
        }
        __syncthreads();
    }
    }

    int* sl = seglen + (long long)b * nt;
    for (int t = tid; t < nt; t += kThreads) sl[t] = base[t] - rp[t];
}


// ----------------------------------------------------------------------------- 128 rows at a time
// Same scheme as pass 2 above with four rows per warp and 128-bit row masks: a quarter of the
// block-wide barriers.  Needs 9 words of shared memory per target.  m <= 32 P.
constexpr int kR = 4;                    // rows per warp and group
constexpr int kGroupRows = kWarps * kR;  // 128
// M48: m = 48 known at compile time (P = 2)
template <int P, bool M48>
__global__ void __launch_bounds__(kThreads)
inverse_build128_kernel(const int64_t* __restrict__ idx, int n_rows, int m_arg, int nt, int* __restrict__ header,
                        int* __restrict__ rowptr, int* __restrict__ seglen, int* __restrict__ entries,
                        int* __restrict__ tileflag, int ntiles) {
    const int m = M48 ? 48 : m_arg;
    extern __shared__ __align__(16) int sm128[];
    unsigned* mask = reinterpret_cast<unsigned*>(sm128);             // [nt][4] rows of the current group that hit t
    unsigned* dupm = reinterpret_cast<unsigned*>(sm128 + 4 * nt);    // [nt][4] rows that hit t more than once
    int* base = sm128 + 8 * nt;                                      // [nt] running write position of target t
    __shared__ int warp_tot[kWarps];
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long E = (long long)n_rows * m;
    const int64_t* ib = idx + (long long)b * E;
    int* rp = rowptr + (long long)b * (nt + 1);
    int* ent = entries + (long long)b * E;
    if (b == 0 && tid == 0) {
        header[0] = (int)kInvMagic;
        header[1] = gridDim.x;
        header[2] = n_rows;
        header[3] = m;
        header[4] = nt;
    }
    {
        int* tf = tileflag + (long long)b * (1 + ntiles);
        if (tf[0] != kBuildGeneral) return;
        for (int t = tid; t < ntiles; t += kThreads) tf[1 + t] = kTileGeneral;
    }
    for (int t = tid; t < nt; t += kThreads) base[t] = 0;
    for (int t = tid; t < 4 * nt; t += kThreads) {
        mask[t] = 0u;
        dupm[t] = 0u;
    }
    __syncthreads();
    int oob = 0;
    {
        // eight indices per thread in flight at a time
        constexpr int kBatch = 8;
        for (long long e0 = tid; e0 < E; e0 += (long long)kBatch * kThreads) {
            long long tk[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const long long e = e0 + (long long)u * kThreads;
                tk[u] = e < E ? ib[e] : 0;
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const long long e = e0 + (long long)u * kThreads;
                if (e < E) {
                    if (tk[u] >= 0 && tk[u] < nt) atomicAdd(&base[(int)tk[u]], 1);
                    else ++oob;
                }
            }
        }
    }
    if (oob) atomicAdd(&header[5], oob);
    __syncthreads();
    {
        const int per = (nt + kThreads - 1) / kThreads;
        const int lo = min(tid * per, nt);
        const int hi = min(lo + per, nt);
        int local = 0;
        for (int t = lo; t < hi; ++t) local += base[t];
        int incl = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int y = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += y;
        }
        if (lane == 31) warp_tot[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            const int w = warp_tot[lane];
            int wi = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int y = __shfl_up_sync(0xffffffffu, wi, o);
                if (lane >= o) wi += y;
            }
            warp_tot[lane] = wi - w;
        }
        __syncthreads();
        int run = warp_tot[warp] + incl - local;
        for (int t = lo; t < hi; ++t) {
            const int cnt = base[t];
            base[t] = run;
            rp[t] = run;
            run += cnt;
        }
        if (hi == nt && lo < nt) rp[nt] = run;
        if (nt == 0 && tid == 0) rp[0] = 0;
    }
    __syncthreads();

    // row g0 + 4 warp + r of a group is bit (4 warp + r) % 32 of mask word warp / 8
    const int word = warp >> 3;
    const int bit0 = (warp & 7) * kR;
    int cur[kR][P], nxt[kR][P];
    auto load_rows = [&](int row0, int (&dst)[kR][P]) {
#pragma unroll
        for (int r = 0; r < kR; ++r)
#pragma unroll
            for (int p = 0; p < P; ++p) {
                const int j = lane + 32 * p;
                long long tk = -1;
                // volatile: the loads of the next group are issued here, ahead of this group's barriers
                if (row0 + r < n_rows && j < m)
                    asm volatile("ld.global.nc.s64 %0, [%1];\n" : "=l"(tk) : "l"(ib + (long long)(row0 + r) * m + j));
                dst[r][p] = (tk >= 0 && tk < nt) ? (int)tk : -1;
            }
    };
    load_rows(warp * kR, cur);
    for (int g0 = 0; g0 < n_rows; g0 += kGroupRows) {
        const int row0 = g0 + warp * kR;
        load_rows(row0 + kGroupRows, nxt);
        unsigned win = 0u, last = 0u;                     // bit r * P + p
        // The warp's four rows are often one and the same neighbour list (the tokens of a cluster share
        // theirs): they are then marked with one atomic per slot and placed at four consecutive positions.
        bool same4 = row0 + kR <= n_rows;
#pragma unroll
        for (int p = 0; p < P; ++p)
            same4 = same4 && cur[0][p] == cur[1][p] && cur[0][p] == cur[2][p] && cur[0][p] == cur[3][p];
        same4 = __all_sync(0xffffffffu, same4);
        if (same4) {
            const unsigned bits = 0xfu << bit0, first = 1u << bit0;
#pragma unroll
            for (int p = 0; p < P; ++p)
                if (cur[0][p] >= 0) {
                    const unsigned old = atomicOr(&mask[cur[0][p] * 4 + word], bits);
                    if (old & first) atomicOr(&dupm[cur[0][p] * 4 + word], bits);
                    else win |= 1u << p;
                }
        } else {
#pragma unroll
            for (int r = 0; r < kR; ++r)
#pragma unroll
                for (int p = 0; p < P; ++p)
                    if (cur[r][p] >= 0) {
                        const unsigned bit = 1u << (bit0 + r);
                        const unsigned old = atomicOr(&mask[cur[r][p] * 4 + word], bit);
                        if (old & bit) atomicOr(&dupm[cur[r][p] * 4 + word], bit);
                        else win |= 1u << (r * P + p);
                    }
        }
        __syncthreads();
        if (same4) {
#pragma unroll
            for (int p = 0; p < P; ++p)
                if ((win >> p) & 1u) {
                    const int tk = cur[0][p];
                    const uint4 mk = *reinterpret_cast<const uint4*>(&mask[tk * 4]);
                    const unsigned mw[4] = {mk.x, mk.y, mk.z, mk.w};
                    const unsigned first = 1u << bit0;
                    int pos = base[tk];
                    bool later = false;                   // does a later row of the group hit tk too?
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        if (w < word) pos += __popc(mw[w]);
                        else if (w == word) {
                            pos += __popc(mw[w] & (first - 1u));
                            later = later || (bit0 + kR < 32 && (mw[w] >> (bit0 + kR)) != 0u);
                        } else {
                            later = later || mw[w] != 0u;
                        }
                    }
                    const bool dup = (dupm[tk * 4 + word] & first) != 0u;
#pragma unroll
                    for (int r = 0; r < kR; ++r)
                        ent[pos + r] = dup ? (int)(kDupFlag | (unsigned)((row0 + r) * m)) : ((row0 + r) * m + lane + 32 * p);
                    if (!later) last |= 1u << p;
                }
        } else {
#pragma unroll
        for (int r = 0; r < kR; ++r)
#pragma unroll
            for (int p = 0; p < P; ++p)
                if ((win >> (r * P + p)) & 1u) {
                    const int tk = cur[r][p];
                    const uint4 mk = *reinterpret_cast<const uint4*>(&mask[tk * 4]);
                    const unsigned mw[4] = {mk.x, mk.y, mk.z, mk.w};
                    const unsigned bit = 1u << (bit0 + r);
                    int pos = base[tk];
                    bool later = false;                   // does a later row of the group hit tk too?
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        if (w < word) pos += __popc(mw[w]);
                        else if (w == word) {
                            pos += __popc(mw[w] & (bit - 1u));
                            later = later || (mw[w] >> (bit0 + r)) != 1u;
                        } else {
                            later = later || mw[w] != 0u;
                        }
                    }
                    const bool dup = (dupm[tk * 4 + word] & bit) != 0u;
                    const int row = row0 + r;
                    ent[pos] = dup ? (int)(kDupFlag | (unsigned)(row * m)) : (row * m + lane + 32 * p);
                    if (!later) last |= 1u << (r * P + p);
                }
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < kR; ++r)
#pragma unroll
            for (int p = 0; p < P; ++p)
                if ((last >> (r * P + p)) & 1u) {
                    const int tk = cur[r][p];
                    const uint4 mk = *reinterpret_cast<const uint4*>(&mask[tk * 4]);
                    base[tk] += __popc(mk.x) + __popc(mk.y) + __popc(mk.z) + __popc(mk.w);
                    *reinterpret_cast<uint4*>(&mask[tk * 4]) = make_uint4(0u, 0u, 0u, 0u);
                    *reinterpret_cast<uint4*>(&dupm[tk * 4]) = make_uint4(0u, 0u, 0u, 0u);
                }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < kR; ++r)
#pragma unroll
            for (int p = 0; p < P; ++p) cur[r][p] = nxt[r][p];
    }
    int* sl = seglen + (long long)b * nt;
    for (int t = tid; t < nt; t += kThreads) sl[t] = base[t] - rp[t];
}

}  // namespace

int launch_inverse_build(const int64_t* idx, int b, int n_rows, int m, int nt, void* buf, cudaStream_t s) {
    int* p = static_cast<int*>(buf);
    InverseView v = inverse_view(buf, b, n_rows, m, nt);
    if (cudaMemsetAsync(p, 0, kInvHeaderInts * sizeof(int), s) != cudaSuccess) {
        cudaGetLastError();
        return CLUSTEN_ERR_CUDA;
    }
    // structured tables first; what that build did not take is done below
    {
        const int st = launch_inverse_struct(idx, b, n_rows, m, nt, buf, s);
        if (st != CLUSTEN_OK) return st;
    }
    if (m <= 64 && size_t(9) * nt * sizeof(int) <= 200 * 1024) {
        const size_t smem128 = size_t(9) * nt * sizeof(int);
        auto kernel128 = m == 48 ? inverse_build128_kernel<2, true>
                                 : (m <= 32 ? inverse_build128_kernel<1, false> : inverse_build128_kernel<2, false>);
        const int fit = resident_ctas(reinterpret_cast<const void*>(kernel128), kThreads, smem128);
        if (fit < 0) return fit;
        ScopedKernelTimer timer("inverse_build", s);
        kernel128<<<b, kThreads, smem128, s>>>(idx, n_rows, m, nt, p, const_cast<int*>(v.rowptr),
                                               const_cast<int*>(v.seglen), const_cast<int*>(v.entries),
                                               const_cast<int*>(v.tileflag), v.ntiles);
        note_launch();
        return check_launch();
    }
    int* scratch = nullptr;
    if (nt > kInvSmemTargets)
        scratch = const_cast<int*>(v.tileflag) + inv_align(size_t(b) * (1 + v.ntiles));
    const size_t smem = scratch ? 0 : size_t(3) * nt * sizeof(int);
    auto kernel = m <= 32 ? inverse_build_kernel<1> : (m <= 64 ? inverse_build_kernel<2> : inverse_build_kernel<0>);
    const int fit = resident_ctas(reinterpret_cast<const void*>(kernel), kThreads, smem);
    if (fit < 0) return fit;
    ScopedKernelTimer timer("inverse_build", s);
    kernel<<<b, kThreads, smem, s>>>(idx, n_rows, m, nt, p, const_cast<int*>(v.rowptr),
                                     const_cast<int*>(v.seglen), const_cast<int*>(v.entries), scratch,
                                     const_cast<int*>(v.tileflag), v.ntiles);
    note_launch();
    return check_launch();
}

}  // namespace clusten
