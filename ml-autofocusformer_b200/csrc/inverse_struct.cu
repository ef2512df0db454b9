// Inverse neighbour index for STRUCTURED neighbour tables, 8 indices at a time.
//
// AutoFocusFormer's tables are never arbitrary.  Either the 8 tokens of a cluster share one row
// ("clusters": rows 8c .. 8c+7 of nbhd_idx are identical), or every row is a concatenation of whole
// clusters ("runs": each aligned group of 8 slots holds the tokens 8T .. 8T+7, which is what
// models/aff_transformer.py:476-482 of the reference builds from models/point_utils.py:203-206).
// In both cases the inverse of a batch element has an eighth of the degrees of freedom:
//
//   clusters   target t is named by (cluster c, slot j); its segment is the 8 rows of c, one after
//              the other, for every such pair
//   runs       target run T is named by (row i, run slot jr); the segments of its 8 targets list the
//              same rows in the same order, target 8T+q at slot 8 jr + q
//
// One CTA per batch element checks which of the two holds (reading every index once), counts and places
// the (c, j) or (i, jr) pairs with integer atomics in shared memory, sorts each short list (so that the
// result does not depend on the order of the atomics) and expands it into the per-target segments of the
// general format (common.cuh).  It also records, per tile of 8 targets, that the tile is structured,
// which lets the scatter-side kernels skip their own analysis.  Batch elements that are neither (random
// rows, out-of-range indices, padded tails) are left to the general build (inverse.cu).
#include <limits.h>

#include "common.cuh"

namespace clusten {
namespace {

constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;
constexpr unsigned kFull = 0xffffffffu;
constexpr int kShortList = 24;           // lists up to this length are sorted by one thread
constexpr int kQueue = 1024;             // longer lists wait here for a whole warp

// exclusive scan of cnt[0..N) into out[0..N); returns the total in every thread.  All threads call it.
__device__ int block_exclusive_scan(const int* cnt, int* out, int N, int* warp_tot) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int per = (N + kThreads - 1) / kThreads;
    const int lo = min(tid * per, N), hi = min(lo + per, N);
    int local = 0;
    for (int t = lo; t < hi; ++t) local += cnt[t];
    int incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(kFull, incl, o);
        if (lane >= o) incl += y;
    }
    __syncthreads();                       // warp_tot may still be read from an earlier call
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const int w = warp_tot[lane];
        int wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int y = __shfl_up_sync(kFull, wi, o);
            if (lane >= o) wi += y;
        }
        warp_tot[lane] = wi - w;
        if (lane == 31) warp_tot[32] = wi;
    }
    __syncthreads();
    int run = warp_tot[warp] + incl - local;
    for (int t = lo; t < hi; ++t) {
        const int c = cnt[t];
        out[t] = run;
        run += c;
    }
    const int total = warp_tot[32];
    __syncthreads();
    return total;
}

// ascending sort of a[0..L) by one warp, any L: the bitonic network in the form whose every
// compare-exchange moves the smaller value to the lower position, so positions past L can stand for
// +infinity and are simply never touched
__device__ void warp_sort_smem(unsigned short* a, int L, int lane) {
    int P = 2;
    while (P < L) P <<= 1;
    auto pass = [&](int mask_or_j, bool flip) {
        for (int i = lane; i < P; i += 32) {
            const int l = flip ? (i ^ mask_or_j) : (i ^ mask_or_j);
            if (l > i && l < L) {
                const unsigned short x = a[i], y = a[l];
                if (x > y) {
                    a[i] = y;
                    a[l] = x;
                }
            }
        }
        __syncwarp();
    };
    for (int k = 2; k <= P; k <<= 1) {
        pass(k - 1, true);                                 // partner: mirror image inside the block of k
        for (int j = k >> 2; j > 0; j >>= 1) pass(j, false);
    }
}

}  // namespace

// P = passes of 32 slots over a row (m <= 32 P)
template <int P>
__global__ void __launch_bounds__(kThreads)
inverse_struct_kernel(const int64_t* __restrict__ idx, int n_rows, int m, int nt, int ntiles, int max_tile_pairs,
                      unsigned m_magic, unsigned m_shift, int with_owner, int warp_counts, int* __restrict__ header, int* __restrict__ rowptr, int* __restrict__ seglen,
                      int* __restrict__ entries, int* __restrict__ tileflag) {
    extern __shared__ __align__(16) int sm[];
    int* cntS = sm;                                   // [nt]      pairs per target (clusters)
    int* cntM = cntS + nt;                            // [ntiles]  pairs per target run (runs)
    int* cur = cntM + ntiles;                         // [nt]      write cursor of the chosen kind
    unsigned short* placed = reinterpret_cast<unsigned short*>(cur + nt);    // [n_rows * m / 8] the pairs, by target
    // the target (clusters) or target run (runs) of every placed pair, when shared memory has room for it (a
    // search in cur otherwise)
    unsigned short* owner = with_owner ? placed + ((n_rows * m / 8 + 1) & ~1) : nullptr;
    // runs: pairs per (warp, target run), each warp counting the rows it will later place (in order, so that
    // the run's pairs come out sorted without a sort); behind placed / owner when there is room
    int* cntW = warp_counts ? reinterpret_cast<int*>(placed + (with_owner ? 2 : 1) * ((n_rows * m / 8 + 1) & ~1)) : nullptr;
    __shared__ int warp_tot[kWarps + 1];
    __shared__ int ok_clusters, ok_runs, q_len;
    __shared__ int queue[kQueue];

    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long E = (long long)n_rows * m;
    const int64_t* ib = idx + (long long)b * E;
    int* rp = rowptr + (long long)b * (nt + 1);
    int* sl = seglen + (long long)b * nt;
    int* ent = entries + (long long)b * E;
    int* tf = tileflag + (long long)b * (1 + ntiles);
    const int R = m >> 3;                             // run slots per row
    auto div_m = [&](unsigned x) { return (__umulhi(m_magic, x) + x) >> m_shift; };      // x / m for x < 2^31

    if (b == 0 && tid == 0) {
        header[0] = (int)kInvMagic;
        header[1] = gridDim.x;
        header[2] = n_rows;
        header[3] = m;
        header[4] = nt;
    }
    for (int t = tid; t < nt; t += kThreads) cntS[t] = 0;
    for (int t = tid; t < ntiles; t += kThreads) cntM[t] = 0;
    if (cntW)
        for (int t = tid; t < kWarps * ntiles; t += kThreads) cntW[t] = 0;
    if (tid == 0) {
        ok_clusters = (n_rows % 8 == 0) ? 1 : 0;
        ok_runs = (m % 8 == 0) ? 1 : 0;
        q_len = 0;
    }
    __syncthreads();

    // ---- pass 1: every index once; which structure holds, and the counts of both
    {
        bool clusters = true, runs = true;
        const int blocks = (n_rows + 7) >> 3;
        const int per_warp = (blocks + kWarps - 1) / kWarps;           // a contiguous range of row blocks per warp
        int* cnt_runs = cntW ? cntW + warp * ntiles : cntM;
        for (int k = warp * per_warp; k < min(blocks, (warp + 1) * per_warp); ++k) {
            // nothing left to find out once both structures are ruled out (by this warp or another one)
            if (!clusters && !runs) break;
            if (*reinterpret_cast<volatile int*>(&ok_clusters) == 0 && *reinterpret_cast<volatile int*>(&ok_runs) == 0) break;
            int v[8][P];
#pragma unroll
            for (int r = 0; r < 8; ++r)
#pragma unroll
                for (int p = 0; p < P; ++p) {
                    const int j = lane + 32 * p, row = 8 * k + r;
                    unsigned long long tk = ~0ull;
                    if (row < n_rows && j < m) tk = (unsigned long long)__ldg(ib + (long long)row * m + j);
                    v[r][p] = tk < (unsigned long long)nt ? (int)tk : -1;          // negative or too large: -1
                }
            bool same = true, inrange = true;
#pragma unroll
            for (int p = 0; p < P; ++p) {
                const int j = lane + 32 * p;
                if (j < m) {
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        if (8 * k + r < n_rows) {
                            inrange = inrange && v[r][p] >= 0;
                            same = same && v[r][p] == v[0][p];
                        } else {
                            same = false;
                        }
                    }
                }
            }
            same = __all_sync(kFull, same && inrange);
            inrange = __all_sync(kFull, inrange);
            clusters = clusters && same;
            runs = runs && inrange;
            if (same) {
#pragma unroll
                for (int p = 0; p < P; ++p)
                    if (lane + 32 * p < m) atomicAdd(&cntS[v[0][p]], 1);
            }
            if (inrange && (m & 7) == 0 && runs) {
                // is every aligned group of 8 slots one whole cluster 8T .. 8T+7?  Identical rows are checked once.
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    if (r == 0 || !same) {
#pragma unroll
                        for (int p = 0; p < P; ++p) {
                            const int j = lane + 32 * p;
                            const int v0 = __shfl_sync(kFull, v[r][p], lane & ~7);     // slot j & ~7 of the same pass
                            if (j < m && 8 * k + r < n_rows) {
                                const bool good = (v0 & 7) == 0 && v[r][p] == v0 + (lane & 7) && v0 + 7 < nt;
                                runs = runs && good;
                                if (good && (lane & 7) == 0) atomicAdd(&cnt_runs[v0 >> 3], same ? 8 : 1);
                            }
                        }
                    }
                }
                runs = __all_sync(kFull, runs);
            }
            if (!clusters && lane == 0) ok_clusters = 0;
            if (!runs && lane == 0) ok_runs = 0;
        }
        if (!__all_sync(kFull, clusters) && lane == 0) ok_clusters = 0;
        if (!__all_sync(kFull, runs) && lane == 0) ok_runs = 0;
    }
    __syncthreads();
    // codes of the pairs must fit in 16 bits
    const bool fits = (long long)n_rows * m / 8 <= 65535;
    const int mode = !fits ? kBuildGeneral : (ok_runs ? kBuildRuns : (ok_clusters ? kBuildClusters : kBuildGeneral));
    if (mode == kBuildGeneral) {
        if (tid == 0) tf[0] = kBuildGeneral;
        return;
    }

    if (mode == kBuildClusters) {
        // ---- clusters: cur = exclusive scan of cntS (in pairs; a pair is 8 entries)
        const int total = block_exclusive_scan(cntS, cur, nt, warp_tot);
        if (tid == 0) rp[nt] = 8 * total;
        // ---- place the (cluster, slot) pairs: row 8k stands for its cluster; two clusters per warp in flight
        {
            const int nblocks = n_rows >> 3;
            for (int k = warp; k < nblocks; k += 2 * kWarps) {
                int t0[P], t1[P];
                const int k1 = k + kWarps;
#pragma unroll
                for (int p = 0; p < P; ++p) {
                    const int j = lane + 32 * p;
                    t0[p] = j < m ? (int)__ldg(ib + (long long)(8 * k) * m + j) : -1;
                    t1[p] = (j < m && k1 < nblocks) ? (int)__ldg(ib + (long long)(8 * k1) * m + j) : -1;
                }
#pragma unroll
                for (int p = 0; p < P; ++p) {
                    const int j = lane + 32 * p;
                    if (t0[p] >= 0) {
                        const int pos = atomicAdd(&cur[t0[p]], 1);
                        placed[pos] = (unsigned short)(k * m + j);
                        if (owner) owner[pos] = (unsigned short)t0[p];
                    }
                    if (t1[p] >= 0) {
                        const int pos = atomicAdd(&cur[t1[p]], 1);
                        placed[pos] = (unsigned short)(k1 * m + j);
                        if (owner) owner[pos] = (unsigned short)t1[p];
                    }
                }
            }
        }
        __syncthreads();
        // cur[t] is now the END of target t's pairs; cntS[t] their number.  Bit 30 of cntS[t] will say that the
        // segment needs the slow path: a cluster names t more than once, or the list is long.
        constexpr int kSlow = 1 << 30;
        constexpr int kLong = 64;
        // ---- one thread per pair: its rank among the target's pairs is where its 8 entries go (the rows of
        //      its cluster at its slot, 32 contiguous bytes), so the segment comes out ordered by row whatever
        //      order the atomics ran in
        for (int p = tid; p < total; p += kThreads) {
            int t;
            if (owner) {
                t = owner[p];
            } else {
                int lo = 0, hi = nt - 1;              // the first target whose pairs end behind p
                while (lo < hi) {
                    const int mid = (lo + hi) >> 1;
                    if (cur[mid] > p) hi = mid;
                    else lo = mid + 1;
                }
                t = lo;
            }
            const int L = cntS[t] & ~kSlow, b0 = cur[t] - L;
            if (L > kLong) {
                if (p == b0) atomicOr(&cntS[t], kSlow);
                continue;
            }
            const unsigned code = placed[p];
            const unsigned c = div_m(code), j = code - c * (unsigned)m;
            int rank = 0;
            bool repeat = false;
            for (int i = 0; i < L; ++i) {
                const unsigned other = placed[b0 + i];
                rank += other < code ? 1 : 0;
                repeat = repeat || (other != code && div_m(other) == c);
            }
            if (repeat) atomicOr(&cntS[t], kSlow);
            const int e0 = (int)(8u * c * (unsigned)m + j);
            int* dst = ent + 8 * (long long)(b0 + rank);
            *reinterpret_cast<int4*>(dst) = make_int4(e0, e0 + m, e0 + 2 * m, e0 + 3 * m);
            *reinterpret_cast<int4*>(dst + 4) = make_int4(e0 + 4 * m, e0 + 5 * m, e0 + 6 * m, e0 + 7 * m);
        }
        __syncthreads();
        // ---- segment starts and lengths; the slow targets go to a queue
        for (int t = tid; t < nt; t += kThreads) {
            const int Lr = cntS[t], L = Lr & ~kSlow;
            rp[t] = 8 * (cur[t] - L);
            if (!(Lr & kSlow)) {
                sl[t] = 8 * L;
            } else {
                const int slot = atomicAdd(&q_len, 1);
                if (slot < kQueue) queue[slot] = t;
                else cntS[t] = Lr | (1 << 29);                      // no room: this thread does it itself below
            }
        }
        __syncthreads();
        // ---- slow targets, one warp each: sort, then one group of entries per distinct cluster -- its 8 rows
        //      at the pair's slot, or flagged rows when the cluster names the target more than once
        auto slow_target = [&](int t, int sub, int nsub) {            // nsub = 32: a warp; nsub = 1: one thread
            const int L = cntS[t] & ((1 << 29) - 1), b0 = cur[t] - L;
            unsigned short* a = placed + b0;
            if (nsub == 32) {
                warp_sort_smem(a, L, sub);
            } else {
                for (int i = 1; i < L; ++i) {
                    const unsigned short x = a[i];
                    int j = i - 1;
                    while (j >= 0 && a[j] > x) {
                        a[j + 1] = a[j];
                        --j;
                    }
                    a[j + 1] = x;
                }
            }
            int* dst = ent + 8 * (long long)b0;
            int d_base = 0;
            for (int i0 = 0; i0 < L; i0 += nsub) {
                const int i = i0 + sub;
                const unsigned code = i < L ? a[i] : 0u;
                const int c = i < L ? (int)div_m(code) : -1;
                const int pc = (i > 0 && i < L) ? (int)div_m(a[i - 1]) : -1;
                const int nc = i + 1 < L ? (int)div_m(a[i + 1]) : -2;
                const bool first = i < L && c != pc;
                const unsigned mk = nsub == 32 ? __ballot_sync(kFull, first) : (first ? 1u : 0u);
                if (first) {
                    const int d = d_base + __popc(mk & ((1u << sub) - 1u));
                    int e0 = (int)(8u * (unsigned)c * (unsigned)m + (code - (unsigned)c * (unsigned)m));
                    if (nc == c) e0 = (int)(kDupFlag | (8u * (unsigned)c * (unsigned)m));
                    *reinterpret_cast<int4*>(dst + 8 * d) = make_int4(e0, e0 + m, e0 + 2 * m, e0 + 3 * m);
                    *reinterpret_cast<int4*>(dst + 8 * d + 4) = make_int4(e0 + 4 * m, e0 + 5 * m, e0 + 6 * m, e0 + 7 * m);
                }
                d_base += __popc(mk);
            }
            if (sub == 0) sl[t] = 8 * d_base;
        };
        {
            const int nq = min(q_len, kQueue);
            for (int qi = warp; qi < nq; qi += kWarps) slow_target(queue[qi], lane, 32);
            if (q_len > kQueue)
                for (int t = tid; t < nt; t += kThreads)
                    if (cntS[t] & (1 << 29)) slow_target(t, 0, 1);
        }
        // ---- tiles: structured when complete, without slow targets and small enough for the lean kernel
        for (int T = tid; T < ntiles; T += kThreads) {
            bool ok = 8 * T + 8 <= nt;
            int pairs = 0;
            if (ok) {
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const int Lr = cntS[8 * T + q];
                    ok = ok && !(Lr & kSlow);
                    pairs += Lr & ((1 << 29) - 1);
                }
            }
            tf[1 + T] = (ok && pairs <= max_tile_pairs) ? kTileClusters : kTileGeneral;
        }
        if (tid == 0) tf[0] = kBuildClusters;
        return;
    }

    // ---- runs (a pair is one entry for each of the run's 8 targets)
    constexpr int kSlowRun = 1 << 30;
    unsigned r_shift = 0;                             // x / R for x < 2^31 (R <= 8)
    while ((1u << r_shift) < (unsigned)R) ++r_shift;
    const unsigned r_magic = (unsigned)(((1ull << 32) * ((1ull << r_shift) - (unsigned)R)) / (unsigned)R + 1);
    auto div_R = [&](unsigned x) { return (__umulhi(r_magic, x) + x) >> r_shift; };
    if (cntW) {
        for (int T = tid; T < ntiles; T += kThreads) {
            int tot = 0;
            for (int w = 0; w < kWarps; ++w) tot += cntW[w * ntiles + T];
            cntM[T] = tot;
        }
        __syncthreads();
    }
    const int total = block_exclusive_scan(cntM, cur, ntiles, warp_tot);     // cur[T]: start of run T's pairs
    if (tid == 0) rp[nt] = 8 * total;
    if (cntW) {
        // start of every warp's share of every run
        for (int T = tid; T < ntiles; T += kThreads) {
            int running = cur[T];
            for (int w = 0; w < kWarps; ++w) {
                const int c = cntW[w * ntiles + T];
                cntW[w * ntiles + T] = running;
                running += c;
            }
            cur[T] = running;                          // end of the run's pairs, as after an atomic placement
        }
        __syncthreads();
        // ---- ordered placement: every warp walks its rows in ascending order, a few rows per trip; pairs of one
        //      trip that name the same run are ranked by lane (= by row, then slot)
        const int rows_per = 32 / R;
        const int sub = lane / R, jr = lane - sub * R;
        const int blocks = (n_rows + 7) >> 3;
        const int per_warp = (blocks + kWarps - 1) / kWarps;
        const int row_lo = min(n_rows, 8 * warp * per_warp), row_hi = min(n_rows, 8 * (warp + 1) * per_warp);
        int* mine = cntW + warp * ntiles;
        for (int r0 = row_lo; r0 < row_hi; r0 += rows_per) {
            const int row = r0 + sub;
            const bool act = sub < rows_per && row < row_hi;
            const int T = act ? (int)(__ldg(ib + (long long)row * m + 8 * jr) >> 3) : -1 - lane;
            const unsigned peers = __match_any_sync(kFull, T);
            const int before = __popc(peers & ((1u << lane) - 1u));
            int pos = 0;
            if (act) pos = mine[T] + before;
            __syncwarp();
            if (act) {
                if (before == 0) mine[T] += __popc(peers);
                placed[pos] = (unsigned short)(row * R + jr);
                if (owner) owner[pos] = (unsigned short)T;
                // a row that names the run twice: two peers inside the row's own lanes
                const unsigned rowmask = ((R == 32 ? 0xffffffffu : ((1u << R) - 1u)) << (sub * R));
                if (__popc(peers & rowmask) > 1) atomicOr(&cntM[T], kSlowRun);
            }
            __syncwarp();
        }
        __syncthreads();
        // ---- one thread per pair: the pairs are in order, pair k of a run is entry k of its 8 segments
        for (int p = tid; p < total; p += kThreads) {
            int T;
            if (owner) {
                T = owner[p];
            } else {
                int lo = 0, hi = ntiles - 1;
                while (lo < hi) {
                    const int mid = (lo + hi) >> 1;
                    if (cur[mid] > p) hi = mid;
                    else lo = mid + 1;
                }
                T = lo;
            }
            const int L = cntM[T] & ~kSlowRun, b0 = cur[T] - L;
            const unsigned code = placed[p];
            const unsigned row = div_R(code), jr2 = code - row * (unsigned)R;
            const int nq = min(8, nt - 8 * T);
            const int e0 = (int)(row * (unsigned)m + 8u * jr2);
            int* dst = ent + 8 * (long long)b0 + (p - b0);
            for (int q = 0; q < nq; ++q) dst[q * L] = e0 + q;
        }
    } else {
    {
        const int rows_per = 32 / R;                  // rows per warp and trip, R lanes each
        const int sub = lane / R, jr = lane - sub * R;
        const int trips = (n_rows + rows_per - 1) / rows_per;
        for (int k = warp; k < trips; k += kWarps) {
            const int row = k * rows_per + sub;
            if (sub < rows_per && row < n_rows) {
                const int T = (int)(__ldg(ib + (long long)row * m + 8 * jr) >> 3);
                const int pos = atomicAdd(&cur[T], 1);
                placed[pos] = (unsigned short)(row * R + jr);
                if (owner) owner[pos] = (unsigned short)T;
            }
        }
    }
    __syncthreads();
    // ---- one thread per pair: its rank among the run's pairs is its place in each of the 8 segments
    for (int p = tid; p < total; p += kThreads) {
        int T;
        if (owner) {
            T = owner[p];
        } else {
            int lo = 0, hi = ntiles - 1;
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (cur[mid] > p) hi = mid;
                else lo = mid + 1;
            }
            T = lo;
        }
        const int L = cntM[T] & ~kSlowRun, b0 = cur[T] - L;
        const unsigned code = placed[p];
        const unsigned row = div_R(code), jr = code - row * (unsigned)R;
        int rank = 0;
        bool repeat = false;
        for (int i = 0; i < L; ++i) {
            const unsigned other = placed[b0 + i];
            rank += other < code ? 1 : 0;
            repeat = repeat || (other != code && div_R(other) == row);
        }
        if (repeat) atomicOr(&cntM[T], kSlowRun);
        const int nq = min(8, nt - 8 * T);            // targets of this run that exist
        const int e0 = (int)(row * (unsigned)m + 8u * jr);
        int* dst = ent + 8 * (long long)b0 + rank;
        for (int q = 0; q < nq; ++q) dst[q * L] = e0 + q;
    }
    }
    __syncthreads();
    // ---- per run: segment starts and lengths, the tile's flag; runs that some row names twice are redone
    //      by a warp: sorted, with one flagged entry per such row and target
    for (int T = tid; T < ntiles; T += kThreads) {
        const int Lr = cntM[T], L = Lr & ~kSlowRun, b0 = cur[T] - L;
        const int nq = min(8, nt - 8 * T);
        for (int q = 0; q < nq; ++q) {
            rp[8 * T + q] = 8 * b0 + q * L;
            sl[8 * T + q] = L;
        }
        tf[1 + T] = (!(Lr & kSlowRun) && nq == 8) ? kTileRuns : kTileGeneral;
        if (Lr & kSlowRun) {
            const int slot = atomicAdd(&q_len, 1);
            if (slot < kQueue) queue[slot] = T;
        }
    }
    __syncthreads();
    // (a table with more than kQueue such runs in one batch element is handled run by run)
    const int nslow = q_len;
    for (int qi = warp; qi < (nslow <= kQueue ? nslow : ntiles); qi += kWarps) {
        const int T = nslow <= kQueue ? queue[qi] : qi;
        if (!(cntM[T] & kSlowRun)) continue;
        const int L = cntM[T] & ~kSlowRun, b0 = cur[T] - L;
        unsigned short* a = placed + b0;
        warp_sort_smem(a, L, lane);
        const int nq = min(8, nt - 8 * T);
        int d_base = 0;
        for (int i0 = 0; i0 < L; i0 += 32) {
            const int i = i0 + lane;
            const unsigned code = i < L ? a[i] : 0u;
            const int row = i < L ? (int)div_R(code) : -1;
            const int prow = (i > 0 && i < L) ? (int)div_R(a[i - 1]) : -1;
            const int nrow = i + 1 < L ? (int)div_R(a[i + 1]) : -2;
            const bool first = i < L && row != prow;
            const unsigned mk = __ballot_sync(kFull, first);
            if (first) {
                const int d = d_base + __popc(mk & ((1u << lane) - 1u));
                for (int q = 0; q < nq; ++q)
                    ent[8 * (long long)b0 + q * L + d] = nrow == row ? (int)(kDupFlag | (unsigned)(row * m))
                                                                     : row * m + 8 * (int)(code - (unsigned)row * (unsigned)R) + q;
            }
            d_base += __popc(mk);
        }
        if (lane == 0)
            for (int q = 0; q < nq; ++q) sl[8 * T + q] = d_base;
    }
    if (tid == 0) tf[0] = kBuildRuns;
}

// Launches the structured build for every batch element; tileflag[b][0] tells afterwards which elements
// it handled.  Returns CLUSTEN_OK also when the sizes rule it out (the flags then say "general").
int launch_inverse_struct(const int64_t* idx, int b, int n_rows, int m, int nt, void* buf, cudaStream_t s) {
    int* p = static_cast<int*>(buf);
    InverseView v = inverse_view(buf, b, n_rows, m, nt);
    const int ntiles = inverse_tiles(nt);
    int* tf = const_cast<int*>(v.tileflag);
    const size_t units2 = ((size_t(n_rows) * m / 8 + 1) & ~size_t(1)) * sizeof(unsigned short);
    size_t smem = size_t(2 * nt + ntiles) * sizeof(int) + units2;
    const int with_owner = (nt <= 65535 && smem + units2 <= 200 * 1024) ? 1 : 0;
    if (with_owner) smem += units2;
    const size_t per_warp_counts = size_t(kWarps) * ntiles * sizeof(int);
    const int warp_counts = (m % 8 == 0 && smem + per_warp_counts <= 200 * 1024) ? 1 : 0;
    if (warp_counts) smem += per_warp_counts;
    const bool possible = m <= 64 && smem <= 200 * 1024 && (long long)n_rows * m / 8 <= 65535 &&
                          (m % 8 == 0 || n_rows % 8 == 0);
    if (!possible) {
        // every batch element and tile is "general"
        if (cudaMemsetAsync(tf, 0, size_t(b) * (1 + ntiles) * sizeof(int), s) != cudaSuccess) {
            cudaGetLastError();
            return CLUSTEN_ERR_CUDA;
        }
        return CLUSTEN_OK;
    }
    auto kernel = m <= 32 ? inverse_struct_kernel<1> : inverse_struct_kernel<2>;
    const int fit = resident_ctas(reinterpret_cast<const void*>(kernel), kThreads, smem);
    if (fit < 0) return fit;
    ScopedKernelTimer timer(split_timing_labels() ? "inverse_struct" : "inverse_build", s);
    unsigned m_magic, m_shift = 0;
    while ((1ull << m_shift) < (unsigned)m) ++m_shift;
    m_magic = (unsigned)(((1ull << 32) * ((1ull << m_shift) - (unsigned)m)) / (unsigned)m + 1);
    kernel<<<b, kThreads, smem, s>>>(idx, n_rows, m, nt, ntiles, kStructMaxPairs, m_magic, m_shift, with_owner, warp_counts, p, const_cast<int*>(v.rowptr),
                                     const_cast<int*>(v.seglen), const_cast<int*>(v.entries), tf);
    note_launch();
    return check_launch();
}

}  // namespace clusten
