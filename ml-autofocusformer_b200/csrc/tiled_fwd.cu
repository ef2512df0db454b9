// Tiled kernels for QK / AV (head_dim 32, m <= 48):
//
//   tiled_sum      out[i,:] = sum_j W[i,j] * X[idx[i,j],:]          AV forward, d_query
//   tiled_dot      out[i,j] = <X[idx[i,j],:], Y[i,:]>               QK forward, d_attn
//   tiled_scatter  out[t,:] = sum_{idx[i,j]=t} W[i,j] * X[i,:]      d_key, d_value (over the inverse index)
//
// Every WARP works on its own: it takes a tile of 8 consecutive rows (one AutoFocusFormer
// cluster) of one batch element, reads the tile's int64 neighbour indices once (cp.async into
// shared memory) and then serves all heads from them.  For a head it stages each distinct
// neighbour row ONCE in shared memory (cp.async, 16-byte chunks XOR-swizzled by row) and
// multiplies the 8 rows of the tile against the staged rows on the tensor cores (mma.sync:
// TF32 with a three-pass split for FP32 inputs, m16n8k16 for FP16 / BF16 inputs).  There is no
// block-level synchronisation; latency is hidden by running 16 to 20 such warps per SM (9 to 14 KB
// of shared memory each) and by L2 prefetches of the next tile's index and weight lines.
//
// Tiles whose 8 rows are identical (the tokens of a cluster share their neighbourhood) need no
// de-duplication: the slot of a neighbour is its column.  Otherwise the warp de-duplicates the
// 8 x m indices with a bitmap over token ids (slots ascend with the token id, which fixes the
// summation order) and spreads the weights into a dense [8 x U] matrix, 48 distinct neighbours
// at a time.
//
// The reference gives each output element a thread that re-gathers its neighbour rows from L2
// (clusten/src/clustenav_cuda_kernel.cu:18-50, clustenqk_cuda_kernel.cu:18-49).
#include "tile_core.cuh"

namespace clusten {

namespace {

// Rows that share next to nothing (random tables): staging U rows in rounds of 48 costs more than it
// saves.  Every lane takes one channel and walks the 8 x m edges of the tile directly: the neighbour rows
// come from global memory (contiguous across the warp), the indices are still in the landing area, the
// weights go through shared memory.  Kept out of line so that it does not weigh on the registers of the
// staged path.
// CONTIG: rows 32 elements apart (the [b, h, n, 32] layout), so that a row's offset is a shift
template <typename T, bool CONTIG>
__device__ __noinline__ void gather_sum_unstaged(const long long* ring, float* Wd, const T* __restrict__ A,
                                                 const T* __restrict__ X, T* __restrict__ out, int b, int heads,
                                                 int n, int m, int i0, int lane, long long x_batch, long long x_head,
                                                 int x_row_arg) {
    const int E = kT * m;
    const int4* ring4 = reinterpret_cast<const int4*>(ring);
    const int x_row = CONTIG ? kC : x_row_arg;           // 32 x 32 -> 64-bit products below
    for (int g = 0; g < heads; ++g) {
        const long long bb = (long long)b * heads + g;
        const T* Xh = X + (long long)b * x_batch + (long long)g * x_head + lane;
        const T* Wt = A + (bb * n + i0) * m;
        __syncwarp();
        for (int x = lane; x < E; x += 32) {
            const int q = x / m;
            Wd[x] = i0 + q < n ? Elem<T>::up(Wt[x]) : 0.f;          // [8][m], row stride m
        }
        __syncwarp();
        float accq[kT];
#pragma unroll
        for (int q = 0; q < kT; ++q) accq[q] = 0.f;
        if ((m & 3) == 0) {
#pragma unroll
            for (int q = 0; q < kT; ++q) {
                for (int j = 0; j < m; j += 4) {
                    const float4 w4 = *reinterpret_cast<const float4*>(Wd + q * m + j);
                    const int4 ta = ring4[(q * m + j) >> 1], tb = ring4[((q * m + j) >> 1) + 1];
                    const float wv[4] = {w4.x, w4.y, w4.z, w4.w};
                    const int tl[4] = {ta.x, ta.z, tb.x, tb.z}, th[4] = {ta.y, ta.w, tb.y, tb.w};
                    T xv[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const bool ok = th[e] == 0 && (unsigned)tl[e] < (unsigned)n;
                        xv[e] = ok ? Xh[(long long)tl[e] * x_row] : Elem<T>::down(0.f);
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) accq[q] += wv[e] * Elem<T>::up(xv[e]);
                }
            }
        } else {
#pragma unroll
            for (int q = 0; q < kT; ++q)
                for (int j = 0; j < m; ++j) {
                    const long long t = ring[q * m + j];
                    if (t >= 0 && t < n) accq[q] += Wd[q * m + j] * Elem<T>::up(Xh[(long long)(int)t * x_row]);
                }
        }
#pragma unroll
        for (int q = 0; q < kT; ++q)
            if (i0 + q < n) out[(bb * n + i0 + q) * kC + lane] = Elem<T>::down(accq[q]);
    }
}

// ----------------------------------------------------------------------------- the kernel
// MODE 0: tiled_sum (A = W [bb, n, m]),  MODE 1: tiled_dot (A = Y [bb, n, 32]); X = [bb, n, 32]
// M48: m = 48 (every AutoFocusFormer stage but the last) is known at compile time
template <typename T, int MODE, bool M48>
__global__ void __launch_bounds__(32 * kWarps, MODE == 0 ? 5 : 4)
gather_tiles_kernel(const T* __restrict__ A, const T* __restrict__ X, const int64_t* __restrict__ idx,
                    T* __restrict__ out, int batch, int heads, int n, int m_arg, int tiles, const GatherStrides gs) {
    const int m = M48 ? kMmax : m_arg;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    using WS = WarpSmem<T, MODE>;
    constexpr bool kIsFloat = WS::kIsFloat;
    constexpr int kPer = 16 / (int)sizeof(T);          // elements per 16-byte piece
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int qi = lane >> 3, ci = lane & 7;
    unsigned char* base = smem_raw + size_t(warp) * WS::kTotal;
    float* Xs = reinterpret_cast<float*>(base);
    T* Xraw = reinterpret_cast<T*>(base + WS::kX);
    float* Op = reinterpret_cast<float*>(base + WS::kX + WS::kXraw);
    unsigned short* lut = reinterpret_cast<unsigned short*>(base + WS::kX + WS::kXraw + WS::kOp);
    unsigned short* uniq = lut + kE;
    float* Wd = Op;                                     // MODE 0
    float* Ys = Op;                                     // MODE 1
    float* Sb = Op + kT * kYLD;                         // MODE 1
    long long* ring = reinterpret_cast<long long*>(Xs);               // first 3 KB of X
    DedupScratch ds;
    ds.tok = reinterpret_cast<unsigned short*>(base + kE * 8);        // behind the landed indices
    ds.uniq = uniq;
    ds.bm = reinterpret_cast<unsigned*>(Op);
    ds.pre = reinterpret_cast<unsigned short*>(ds.bm + kBMW);
    ds.rowbm = reinterpret_cast<unsigned*>(ds.pre + kBMW);

    int* tok_s = reinterpret_cast<int*>(uniq);                        // identical rows: source row of X row r
    const SumAddr sa = make_sum_addr(Wd, Xs, lane);                   // MODE 0
    const DotAddr da = make_dot_addr(Ys, Xs, Sb, lane);               // MODE 1

    const int E = kT * m;
    const int m4 = m >> 2;
    // word offset of 16-byte chunk ci inside staged row r = qi + 4k (k even / odd):
    // tiled_sum stores chunk ^ ((r & 3) << 1), tiled_dot chunk ^ (r & 7), see the product routines
    const int sw_even = MODE == 0 ? ((ci ^ (qi << 1)) << 2) : ((ci ^ qi) << 2);
    const int sw_odd = MODE == 0 ? sw_even : (sw_even ^ 16);
    // piece z = lane + 32k of a [8][m] tile -> (row, 4-element piece); edge x = lane + 32k -> its row
    int wq[3], wc[3];
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        const int z = lane + 32 * k;
        const int d = m4 > 0 ? m4 : 1;
        wq[k] = z / d;
        wc[k] = z - wq[k] * d;
    }
    // 16-bit weight tiles travel in 8-element pieces: piece z = lane + 32k of an [8][m] tile, m % 8 == 0
    int wq16[2], wc16[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int z = lane + 32 * k;
        const int d = (m >> 3) > 0 ? (m >> 3) : 1;
        wq16[k] = z / d;
        wc16[k] = z - wq16[k] * d;
    }
    T* Wd16 = reinterpret_cast<T*>(Op);                  // MODE 0, 16-bit inputs: dense weights [8][kWLD16]
    const int col0 = (2 * lane) % m, col_step = 64 % m;
    unsigned long long qpack = 0ull;                    // 3 bits per edge: its row
#pragma unroll
    for (int k = 0; k < kEPL; ++k) qpack |= (unsigned long long)(((lane + 32 * k) / m) & 7) << (3 * k);

    const unsigned total = (unsigned)batch * (unsigned)tiles;       // < 2^31, checked by the launcher
    const unsigned nwarps = gridDim.x * kWarps;
    const unsigned task0 = blockIdx.x * kWarps + warp;
    int b = (int)(task0 / (unsigned)tiles);
    int tile = (int)(task0 - (unsigned)b * (unsigned)tiles);
    const int step_b = (int)(nwarps / (unsigned)tiles), step_t = (int)(nwarps % (unsigned)tiles);
    int nb = b + step_b, ntile = tile + step_t;                      // this warp's next (batch, tile)
    if (ntile >= tiles) { ntile -= tiles; ++nb; }
    for (unsigned task = task0; task < total; task += nwarps) {
        const int i0 = tile * kT;
        const bool complete = i0 + kT <= n;
        const int64_t* src = idx + ((long long)b * n + i0) * m;
        // ---- warm the L2 for this warp's next tile: its index rows and its weight / Y rows
        {
            if (nb < batch) {
                const int ni0 = ntile * kT;
                if (lane * 16 < E) prefetch_l2(idx + ((long long)nb * n + ni0) * m + lane * 16);
                const int arow = MODE == 0 ? m : kC;               // elements per row of A
                const int abytes = kT * arow * (int)sizeof(T);
                const bool a_contig = MODE == 0 || gs.y_row == kC;
                for (int g = 0; g < heads && a_contig; ++g)
                    if (lane * 128 < abytes)
                        prefetch_l2(reinterpret_cast<const char*>(
                                        MODE == 0 ? A + (((long long)nb * heads + g) * n + ni0) * arow
                                                  : A + (long long)nb * gs.y_batch + (long long)g * gs.y_head + (long long)ni0 * gs.y_row) +
                                    lane * 128);
            }
        }
        // ---- the tile's indices
        __syncwarp();
        if (complete && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
            for (int x = 2 * lane; x < E; x += 64) cp_async16_ca(ring + x, src + x);
        } else {
            const int valid = min(kT, n - i0) * m;
            for (int x = lane; x < E; x += 32) {
                if (x < valid) cp_async8_ca(ring + x, src + x);
                else ring[x] = -1;
            }
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncwarp();
        const bool identical = rows_identical(ring, E, m, n, complete, lane, col0, col_step);
        int U = m;
        bool rowdup = false, runs = false;               // runs: lut holds one slot per run of 8 neighbours
        if (identical) {
            const int* ring32 = reinterpret_cast<const int*>(ring);
            for (int r = lane; r < m; r += 32) tok_s[r] = ring32[2 * r];
        } else {
            U = dedup_tile(ds, ring, lut, E, m, i0, n, MODE == 0, &rowdup, lane, -1, &runs);
            if (runs && rowdup) {
                // a row names a run twice: its weights have to be added up, which the per-edge path does
                unsigned short s[kEPL];
#pragma unroll
                for (int k = 0; k < kEPL; ++k) {
                    const int x = lane + 32 * k;
                    s[k] = x < E ? (unsigned short)(lut[x >> 3] * 8 + (x & 7)) : kSkip;
                }
                __syncwarp();
#pragma unroll
                for (int k = 0; k < kEPL; ++k)
                    if (lane + 32 * k < E) lut[lane + 32 * k] = s[k];
                runs = false;
            }
        }
        const int rpr = m >> 3;                          // runs per row (runs tiles have m % 8 == 0)
        __syncwarp();                                    // the landing area is free again
        // 16-bit inputs stay 16-bit (m16n8k16 products) unless a row repeats a neighbour: then the weights
        // of one slot are summed in fp32 and the fp32 path below is taken
        const bool native16 = !kIsFloat && !rowdup;

        if (MODE == 0 && !identical && U > kDirectU) {
            if (gs.x_row == kC)
                gather_sum_unstaged<T, true>(ring, Wd, A, X, out, b, heads, n, m, i0, lane, gs.x_batch, gs.x_head, kC);
            else
                gather_sum_unstaged<T, false>(ring, Wd, A, X, out, b, heads, n, m, i0, lane, gs.x_batch, gs.x_head,
                                              (int)gs.x_row);
            // advance to this warp's next (batch, tile)
            b = nb;
            tile = ntile;
            nb += step_b;
            ntile += step_t;
            if (ntile >= tiles) {
                ntile -= tiles;
                ++nb;
            }
            continue;
        }

        for (int g = 0; g < heads; ++g) {
            const long long bb = (long long)b * heads + g;
            const T* Xh = X + (long long)b * gs.x_batch + (long long)g * gs.x_head;
            const int x_row = (int)gs.x_row;
            float acc[2][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[0][i] = acc[1][i] = 0.f;
            float oreg[kEPL];
#pragma unroll
            for (int k = 0; k < kEPL; ++k) oreg[k] = 0.f;
            unsigned yb16[2][2] = {{0u, 0u}, {0u, 0u}};     // MODE 1, 16-bit inputs: B fragments of the tile's Y rows
            const int nchunks = U > 0 ? (U + kUC - 1) / kUC : 1;
            for (int ch = 0; ch < nchunks; ++ch) {
                const int u0 = ch * kUC;
                const int Uc = max(0, min(kUC, U - u0));
                const int rows8 = (Uc + 7) & ~7;
                __syncwarp();
                // ---- neighbour rows: 8 lanes x 16 bytes per fp32 row (4 lanes per 16-bit row)
                if (kIsFloat && identical) {
                    const T* Xl = Xh + ci * 4;
                    float* dst = Xs + qi * kC;
#pragma unroll
                    for (int k = 0; k < kUC / 4; ++k)
                        if (qi + 4 * k < m)
                            cp_async16_cg(dst + 4 * k * kC + ((k & 1) ? sw_odd : sw_even), Xl + (long long)tok_s[qi + 4 * k] * x_row);
                } else if (kIsFloat) {
#pragma unroll
                    for (int k = 0; k < kUC / 4; ++k) {
                        const int r = qi + 4 * k;
                        if (r < rows8) {
                            int t = -1;
                            if (r < Uc) {
                                if (identical) t = tok_s[r];
                                else {
                                    const unsigned short tt = uniq[u0 + r];
                                    t = tt == kSkip ? -1 : (int)tt;
                                }
                            }
                            float* dst = Xs + r * kC + ((k & 1) ? sw_odd : sw_even);
                            if (t >= 0) cp_async16_cg(dst, Xh + (long long)t * x_row + ci * 4);
                            else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                    }
                } else {
                    const int pr = lane >> 2, pc = lane & 3;
                    const int rows16 = (Uc + 15) & ~15;
#pragma unroll
                    for (int k = 0; k < kUC / 8; ++k) {
                        const int r = pr + 8 * k;
                        if (r < rows16) {
                            int t = -1;
                            if (r < Uc) {
                                if (identical) t = tok_s[r];
                                else {
                                    const unsigned short tt = uniq[u0 + r];
                                    t = tt == kSkip ? -1 : (int)tt;
                                }
                            }
                            T* dst = Xraw + swz16(r, pc);
                            if (t >= 0) cp_async16_cg(dst, Xh + (long long)t * x_row + pc * kPer);
                            else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                    }
                }
                if (MODE == 0) {
                    // ---- weight tile -> Wd while the rows are on their way
                    const T* Wt = A + (bb * n + i0) * m;
                    if (native16 && identical) {
#pragma unroll
                        for (int k = 0; k < 2; ++k)
                            if (lane + 32 * k < kT * (m >> 3))
                                cp_async16_ca(Wd16 + wq16[k] * kWLD16 + wc16[k] * 8, Wt + wq16[k] * m + wc16[k] * 8);
                        if (m & 15) {
                            // the product runs over a multiple of 16 columns: the 8 columns behind the tile are zero
#pragma unroll
                            for (int k = 0; k < 2; ++k) {
                                const int z = lane + 32 * k;
                                Wd16[(z >> 3) * kWLD16 + m + (z & 7)] = Elem<T>::down(0.f);
                            }
                        }
                    } else if (native16 && runs) {
                        // a run's 8 weights of a row are 16 contiguous bytes, and so are its 8 slots
                        for (int z = lane; z < kT * kWLD16 * 2 / 16; z += 32)
                            reinterpret_cast<float4*>(Wd16)[z] = make_float4(0.f, 0.f, 0.f, 0.f);
                        __syncwarp();
                        for (int y = lane; y < kT * rpr; y += 32) {
                            const int q = y / rpr, jr = y - q * rpr;
                            const int rel = (int)lut[y] * 8 - u0;
                            if (rel >= 0 && rel < Uc) cp_async16_ca(Wd16 + q * kWLD16 + rel, Wt + q * m + jr * 8);
                        }
                    } else if (native16) {
                        for (int z = lane; z < kT * kWLD16 * 2 / 16; z += 32)
                            reinterpret_cast<float4*>(Wd16)[z] = make_float4(0.f, 0.f, 0.f, 0.f);
                        __syncwarp();
#pragma unroll
                        for (int k = 0; k < kEPL; ++k) {
                            const int x = lane + 32 * k;
                            if (x < E) {
                                const unsigned short sl = lut[x];
                                const int rel = (int)sl - u0;
                                if (sl != kSkip && rel >= 0 && rel < Uc) {
                                    const int q = (int)((qpack >> (3 * k)) & 7ull);
                                    Wd16[q * kWLD16 + rel] = Wt[x];
                                }
                            }
                        }
                    } else if (identical) {
#pragma unroll
                        for (int k = 0; k < 3; ++k)
                            if (lane + 32 * k < kT * m4) {
                                float* dd = Wd + wq[k] * kWLD + wc[k] * 4;
                                if (kIsFloat) cp_async16_ca(dd, Wt + wq[k] * m + wc[k] * 4);
                                else *reinterpret_cast<float4*>(dd) = ld4(Wt + wq[k] * m + wc[k] * 4);
                            }
                    } else if (runs && kIsFloat) {
                        for (int z = lane; z < kT * kWLD / 4; z += 32)
                            reinterpret_cast<float4*>(Wd)[z] = make_float4(0.f, 0.f, 0.f, 0.f);
                        __syncwarp();
                        for (int y = lane; y < kT * rpr; y += 32) {
                            const int q = y / rpr, jr = y - q * rpr;
                            const int rel = (int)lut[y] * 8 - u0;
                            if (rel >= 0 && rel < Uc) {
                                cp_async16_ca(Wd + q * kWLD + rel, Wt + q * m + jr * 8);
                                cp_async16_ca(Wd + q * kWLD + rel + 4, Wt + q * m + jr * 8 + 4);
                            }
                        }
                    } else {
                        for (int z = lane; z < kT * kWLD / 4; z += 32)
                            reinterpret_cast<float4*>(Wd)[z] = make_float4(0.f, 0.f, 0.f, 0.f);
                        __syncwarp();
                        if (!rowdup) {
#pragma unroll
                            for (int k = 0; k < kEPL; ++k) {
                                const int x = lane + 32 * k;
                                if (x < E) {
                                    const unsigned short sl = lut[x];
                                    const int rel = (int)sl - u0;
                                    if (sl != kSkip && rel >= 0 && rel < Uc) {
                                        const float w = Elem<T>::up(Wt[x]);
                                        const int q = (int)((qpack >> (3 * k)) & 7ull);
                                        Wd[q * kWLD + rel] = w;
                                    }
                                }
                            }
                        } else if (lane < kT) {
                            // some row repeats a neighbour: one lane per row adds the weights in column order
#pragma unroll 1
                            for (int j = 0; j < m; ++j) {
                                const unsigned short sl = lut[lane * m + j];
                                const int rel = (int)sl - u0;
                                if (sl != kSkip && rel >= 0 && rel < Uc) {
                                    Wd[lane * kWLD + rel] += Elem<T>::up(Wt[lane * m + j]);
                                }
                            }
                        }
                    }
                } else if (native16) {
                    // ---- Y tile: the B fragments come straight from global memory, requested here so that they
                    //      arrive together with the staged rows
                    if (ch == 0) {
                        const int yg = lane >> 2, yt = lane & 3;
                        yb16[0][0] = yb16[0][1] = yb16[1][0] = yb16[1][1] = 0u;
                        if (i0 + yg < n) {
                            const unsigned* yrow = reinterpret_cast<const unsigned*>(
                                A + (long long)b * gs.y_batch + (long long)g * gs.y_head + (long long)(i0 + yg) * gs.y_row);
#pragma unroll
                            for (int ks = 0; ks < 2; ++ks) {
                                yb16[ks][0] = yrow[8 * ks + yt];
                                yb16[ks][1] = yrow[8 * ks + 4 + yt];
                            }
                        }
                    }
                } else if (ch == 0) {
                    // ---- Y tile -> Ys (fp32, row stride kYLD)
                    const T* Yt = A + (long long)b * gs.y_batch + (long long)g * gs.y_head + (long long)i0 * gs.y_row;
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const int z = lane + 32 * k;
                        float* dd = Ys + (z >> 3) * kYLD + (z & 7) * 4;
                        const T* ys = Yt + (long long)(z >> 3) * gs.y_row + (z & 7) * 4;
                        if (i0 + (z >> 3) >= n) *reinterpret_cast<float4*>(dd) = make_float4(0.f, 0.f, 0.f, 0.f);
                        else if (kIsFloat) cp_async16_ca(dd, ys);          // lands together with the staged rows
                        else *reinterpret_cast<float4*>(dd) = ld4(ys);
                    }
                }
                cp_async_commit();
                cp_async_wait<0>();
                __syncwarp();
                if (!kIsFloat && !native16) {
                    // 16-bit rows -> fp32, swizzled
#pragma unroll
                    for (int k = 0; k < kUC / 4; ++k) {
                        const int r = qi + 4 * k;
                        if (r < rows8)
                            st4(Xs + r * kC + ((k & 1) ? sw_odd : sw_even), ld4(Xraw + swz16(r, ci >> 1) + (ci & 1) * 4));
                    }
                    __syncwarp();
                }

                if (MODE == 0) {
                    if (native16) sum_product16<T>(Xraw, Wd16, (Uc + 15) >> 4, lane, acc);
                    else sum_product_mma<kIsFloat>(sa, rows8, acc);
                } else {
                    if (native16) {
                        dot_product16<T>(Xraw, yb16, Sb, (Uc + 15) >> 4, lane);
                    } else {
                        dot_product_mma<kIsFloat>(da, (Uc + 15) >> 4);
                    }
                    __syncwarp();
                    T* Ot = out + (bb * n + i0) * m;
                    if (identical) {
#pragma unroll
                        for (int k = 0; k < 3; ++k)
                            if (lane + 32 * k < kT * m4)
                                st4(Ot + wq[k] * m + wc[k] * 4, ld4(Sb + wq[k] * kWLD + wc[k] * 4));
                    } else if (runs) {
                        // the 8 scores of a run of neighbours are neighbours in the score tile and in the output
                        for (int y = lane; y < kT * rpr; y += 32) {
                            const int q = y / rpr, jr = y - q * rpr;
                            const int rel = (int)lut[y] * 8 - u0;
                            if (rel >= 0 && rel < Uc) {
                                st4(Ot + q * m + jr * 8, ld4(Sb + q * kWLD + rel));
                                st4(Ot + q * m + jr * 8 + 4, ld4(Sb + q * kWLD + rel + 4));
                            }
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < kEPL; ++k) {
                            const int x = lane + 32 * k;
                            if (x < E) {
                                const unsigned short sl = lut[x];
                                const int rel = (int)sl - u0;
                                const int q = (int)((qpack >> (3 * k)) & 7ull);
                                if (sl != kSkip && rel >= 0 && rel < Uc) oreg[k] = Sb[q * kWLD + rel];
                            }
                        }
                        if (ch == nchunks - 1) {
#pragma unroll
                            for (int k = 0; k < kEPL; ++k) {
                                const int x = lane + 32 * k;
                                const int q = (int)((qpack >> (3 * k)) & 7ull);
                                if (x < E && i0 + q < n) Ot[x] = Elem<T>::down(oreg[k]);
                            }
                        }
                    }
                }
            }
            if (MODE == 0) {
                // D fragments -> output tile [8][kOLD] in shared memory -> 16-byte stores
                float* Ot = Op;
                const int g = lane >> 2, t = lane & 3;
                __syncwarp();
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    float* o = Ot + (2 * t) * kOLD + 16 * mt + g;
                    o[0] = acc[mt][0];
                    o[kOLD] = acc[mt][1];
                    o[8] = acc[mt][2];
                    o[kOLD + 8] = acc[mt][3];
                }
                __syncwarp();
#pragma unroll
                for (int a = 0; a < 2; ++a) {
                    const int q = 2 * qi + a;
                    if (i0 + q < n)
                        st4(out + (bb * n + i0 + q) * kC + ci * 4,
                            *reinterpret_cast<const float4*>(Ot + q * kOLD + ci * 4));
                }
            }
        }
        // advance to this warp's next (batch, tile)
        b = nb;
        tile = ntile;
        nb += step_b;
        ntile += step_t;
        if (ntile >= tiles) {
            ntile -= tiles;
            ++nb;
        }
    }
}

// ----------------------------------------------------------------------------- scatter side (d_key, d_value, d_feat)
//   out[b, t, 32 s .. 32 s + 31] = sum over inverse-index entries (i, j) of target t and k < ic:
//                                   W[b, s, (i * m + j) * ic + k] * X[b, s, i * ic + k, :]
// Same scheme with targets as tile rows: a warp takes 8 consecutive targets, concatenates their
// inverse-index segments (512 edges at a time), de-duplicates the SOURCE rows, stages each once per
// 32-channel slab ("head") and multiplies the dense [8 x U] weights on the tensor cores.  Segments
// are ordered by source row and slots ascend with the source row, so the summation order is fixed.
// Tiles whose 8 targets are listed by the same rows (neighbourhoods made of whole clusters) skip the
// de-duplication: lane l works for target l % 8, so the 8 weights of one source row, which sit side
// by side in memory, are read by neighbouring lanes.
// QK / AV: ic = 1, a slab is a head.  WF: a slab is 32 of the c channels, the weights are shared by
// the slabs and every entry fans out into its ic (weight, row) pairs.
struct ScatterParams {
    const void* W;  long long w_batch, w_head;                 // element strides
    const void* X;  long long x_batch, x_head;  int x_row;
    void* out;      long long o_batch, o_head;  int o_row;
    const int64_t* idx;  int idx_rows;  int m;                   // nbhd_idx [batch][idx_rows][m]
    InverseView inv;  int n_tgt;
    int ic, heads, batch, tiles;
    int skip_flagged;                                           // tiles the inverse build marked as structured are done elsewhere
    int w_pairs;                                                // W may be read in aligned 32-bit words
    unsigned m_magic, m_shift, ic_magic, ic_shift;              // x / d = (umulhi(magic, x) + x) >> shift
};
__device__ __forceinline__ unsigned fast_div(unsigned x, unsigned magic, unsigned shift) {
    return (__umulhi(magic, x) + x) >> shift;
}

constexpr int kES = 512;            // edges handled at a time (8 targets x ~48 on average)
constexpr unsigned kNoEdge = 0xffffffffu;

template <typename T> struct ScatterSmem {
    static constexpr bool kIsFloat = std::is_same<T, float>::value;
    static constexpr int kX = kUC * kC * 4;         // staged rows; de-duplication scratch before that
    static constexpr int kXraw = kIsFloat ? 0 : kUC * kC * (int)sizeof(T);
    static constexpr int kOp = kT * kWLD * 4;       // dense weights; bitmap scratch; output tile
    static constexpr int kEdge = kES * 4;           // weight index of each edge (bit 31: target repeats in its row)
    static constexpr int kWbuf = kES * 4;           // weight of each edge for the current slab
    static constexpr int kLut = kES * 2;            // slot | tile row << 12;   slot -> source row
    static constexpr int kTotal = kX + kXraw + kOp + kEdge + kWbuf + 2 * kLut;
};
static_assert(2 * kES * 2 <= kUC * kC * 4, "token and slot scratch must fit in the row buffer");

// ATT48: attention tables with m = 48 and ic = 1 (every AutoFocusFormer stage but the last): the divisions by
// m and ic and the edge loops' trip arithmetic are resolved at compile time.
template <typename T, bool ATT48>
__global__ void __launch_bounds__(32 * kWarps, 4)
scatter_tiles_kernel(const ScatterParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    using WS = ScatterSmem<T>;
    constexpr bool kIsFloat = WS::kIsFloat;
    constexpr int kPer = 16 / (int)sizeof(T);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int qi = lane >> 3, ci = lane & 7;
    unsigned char* base = smem_raw + size_t(warp) * WS::kTotal;
    float* Xs = reinterpret_cast<float*>(base);
    T* Xraw = reinterpret_cast<T*>(base + WS::kX);
    float* Wd = reinterpret_cast<float*>(base + WS::kX + WS::kXraw);
    T* Wd16 = reinterpret_cast<T*>(Wd);                          // 16-bit inputs: dense weights [8][kWLD16]
    unsigned* edge = reinterpret_cast<unsigned*>(base + WS::kX + WS::kXraw + WS::kOp);
    float* wbuf = reinterpret_cast<float*>(base + WS::kX + WS::kXraw + WS::kOp + WS::kEdge);
    unsigned short* lut = reinterpret_cast<unsigned short*>(base + WS::kX + WS::kXraw + WS::kOp + WS::kEdge + WS::kWbuf);
    unsigned short* uniq = lut + kES;
    DedupScratch ds;
    ds.tok = reinterpret_cast<unsigned short*>(base);           // the row buffer is free while de-duplicating
    unsigned short* slots = ds.tok + kES;
    ds.uniq = uniq;
    ds.bm = reinterpret_cast<unsigned*>(Wd);
    ds.pre = reinterpret_cast<unsigned short*>(ds.bm + kBMW);
    ds.rowbm = reinterpret_cast<unsigned*>(ds.pre + kBMW);
    const SumAddr sa = make_sum_addr(Wd, Xs, lane);
    const int sw = (ci ^ (qi << 1)) << 2;                       // chunk swizzle of staged row qi + 4k
    const int m = ATT48 ? 48 : p.m, ic = ATT48 ? 1 : p.ic, n_tgt = p.n_tgt;
    const int x_row = ATT48 ? kC : p.x_row, o_row = ATT48 ? kC : p.o_row;      // attention rows are 32 channels
    auto div_m = [&](unsigned x) { return ATT48 ? x / 48u : fast_div(x, p.m_magic, p.m_shift); };
    auto div_ic = [&](unsigned x) { return ATT48 ? x : fast_div(x, p.ic_magic, p.ic_shift); };
    const T* Wg = static_cast<const T*>(p.W);
    const T* Xg = static_cast<const T*>(p.X);
    T* Og = static_cast<T*>(p.out);

    const unsigned total = (unsigned)p.batch * (unsigned)p.tiles;
    const unsigned nwarps = gridDim.x * kWarps;
    // segment (length, start) of target t0 + lane of a task, lanes 0..7
    auto load_segment = [&](unsigned task, int& len, int& start) {
        len = 0;
        start = 0;
        if (task < total) {
            const int b = (int)(task / (unsigned)p.tiles);
            const int tile = (int)(task - (unsigned)b * (unsigned)p.tiles);
            const int t = tile * kT + lane;
            if (p.skip_flagged && p.inv.tileflag[(long long)b * (1 + p.inv.ntiles) + 1 + tile] != kTileGeneral) {
                len = -1;                                       // scatter_struct_kernel has this tile
            } else if (lane < kT && t < n_tgt) {
                len = p.inv.seglen[(long long)b * n_tgt + t];
                start = p.inv.rowptr[(long long)b * (n_tgt + 1) + t];
            }
        }
    };
    int next_len, next_start;
    load_segment(blockIdx.x * kWarps + warp, next_len, next_start);
    const int myq = lane & 7, psub = lane >> 3;
    for (unsigned task = blockIdx.x * kWarps + warp; task < total; task += nwarps) {
        const int b = (int)(task / (unsigned)p.tiles);
        const int t0 = (int)(task - (unsigned)b * (unsigned)p.tiles) * kT;
        const int64_t* idx_b = p.idx + (long long)b * p.idx_rows * m;
        const int* entries = p.inv.entries + (long long)b * p.idx_rows * m;
        const int len = next_len, start = next_start;
        load_segment(task + nwarps, next_len, next_start);      // in flight while this tile is worked on
        if (len < 0) continue;                                  // a structured tile (uniform over the warp)
        const int qlen = __shfl_sync(kFull, len, myq);          // entries of this lane's target
        const int* qent = entries + __shfl_sync(kFull, start, myq);
        int maxlen = len;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) maxlen = max(maxlen, __shfl_xor_sync(kFull, maxlen, o));
        maxlen = __shfl_sync(kFull, maxlen, 0);
        T* Ob = Og + (long long)b * p.o_batch;

        // ---- dense tile back end: the source rows of a pass are in uniq[0 .. Uc), the weight element of
        //      (source row rr, target q) in edge[rr * 8 + q] (kNoEdge: the row does not name the target).
        //      Lane l fills the weights of target l % 8, so the 8 weights of a source row -- neighbours in
        //      memory when the targets are neighbours in the row's list -- are read by neighbouring lanes.
        auto dense_heads = [&](int Uc, bool first) {
            const int rows8 = (Uc + 7) & ~7;
            const int rows16 = (Uc + 15) & ~15;
            for (int g = 0; g < p.heads; ++g) {
                const T* Wh = Wg + (long long)b * p.w_batch + (long long)g * p.w_head;
                const T* Xh = Xg + (long long)b * p.x_batch + (long long)g * p.x_head;
                if (kIsFloat) {
#pragma unroll
                    for (int k = 0; k < kUC / 4; ++k) {
                        const int r = qi + 4 * k;
                        if (r < rows8) {
                            float* dst = Xs + r * kC + sw;
                            if (r < Uc) cp_async16_cg(dst, Xh + (long long)uniq[r] * x_row + ci * 4);
                            else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                    }
                } else {
                    const int pr = lane >> 2, pc = lane & 3;
#pragma unroll
                    for (int k = 0; k < kUC / 8; ++k) {
                        const int r = pr + 8 * k;
                        if (r < rows16) {
                            T* dst = Xraw + swz16(r, pc);
                            if (r < Uc) cp_async16_cg(dst, Xh + (long long)uniq[r] * x_row + pc * kPer);
                            else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                    }
                }
                cp_async_commit();
                if (g == 0 || p.w_head != 0) {
#pragma unroll 4
                    for (int rr = psub; rr < (kIsFloat ? rows8 : rows16); rr += 4) {
                        const unsigned e = rr < Uc ? edge[rr * kT + myq] : kNoEdge;
                        if (kIsFloat) {
                            // asynchronous 4-byte copies, in flight together with the rows staged above
                            float* dst = Wd + myq * kWLD + rr;
                            if (e != kNoEdge) cp_async4_ca(dst, Wh + e);
                            else *dst = 0.f;
                        } else if (p.w_pairs) {
                            // 16-bit weights: the aligned 32-bit word around the element travels; the half is
                            // picked after the wait below
                            if (e != kNoEdge)
                                cp_async4_ca(wbuf + rr * kT + myq,
                                             reinterpret_cast<const void*>(reinterpret_cast<uintptr_t>(Wh + e) & ~uintptr_t(3)));
                        } else {
                            Wd16[myq * kWLD16 + rr] = e != kNoEdge ? Wh[e] : Elem<T>::down(0.f);
                        }
                    }
                    cp_async_commit();
                }
                cp_async_wait<0>();
                __syncwarp();
                if (!kIsFloat && p.w_pairs && (g == 0 || p.w_head != 0)) {
#pragma unroll 4
                    for (int rr = psub; rr < rows16; rr += 4) {
                        const unsigned e = rr < Uc ? edge[rr * kT + myq] : kNoEdge;
                        unsigned short hbits = 0;
                        if (e != kNoEdge) {
                            const unsigned raw = reinterpret_cast<const unsigned*>(wbuf)[rr * kT + myq];
                            hbits = (unsigned short)((reinterpret_cast<uintptr_t>(Wh + e) & 2) ? raw >> 16 : raw & 0xffffu);
                        }
                        reinterpret_cast<unsigned short*>(Wd16)[myq * kWLD16 + rr] = hbits;
                    }
                    __syncwarp();
                }
                float acc[2][4];
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[0][i] = acc[1][i] = 0.f;
                if (kIsFloat) sum_product_mma<true>(sa, rows8, acc);
                else sum_product16<T>(Xraw, Wd16, rows16 >> 4, lane, acc);
                float* Ot = Xs;                                          // the dense weights may serve the next slab
                const int gg = lane >> 2, tt = lane & 3;
                __syncwarp();
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    float* o = Ot + (2 * tt) * kOLD + 16 * mt + gg;
                    o[0] = acc[mt][0];
                    o[kOLD] = acc[mt][1];
                    o[8] = acc[mt][2];
                    o[kOLD + 8] = acc[mt][3];
                }
                __syncwarp();
                T* Oh = Ob + (long long)g * p.o_head;
#pragma unroll
                for (int a = 0; a < 2; ++a) {
                    const int q = 2 * qi + a;
                    if (t0 + q < n_tgt) {
                        T* dstp = Oh + (long long)(t0 + q) * o_row + ci * 4;
                        float4 v = *reinterpret_cast<const float4*>(Ot + q * kOLD + ci * 4);
                        if (!first) {
                            const float4 old = ld4(dstp);
                            v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
                        }
                        st4(dstp, v);
                    }
                }
                __syncwarp();
            }
        };

        // ---- uniform tile: the 8 targets are listed by the same source rows, once each (the 8 tokens of
        //      a cluster always are when neighbourhoods are made of whole clusters).  The dense weights
        //      are then read straight through the entries; nothing to de-duplicate.
        bool uniform = t0 + kT <= n_tgt && maxlen > 0 && ic <= kUC && qlen == maxlen;
        if (__all_sync(kFull, uniform)) {
            for (int r0 = 0; r0 < maxlen; r0 += 4) {                         // all lanes take every trip
                const int r = min(r0 + psub, maxlen - 1);
                const unsigned e = (unsigned)__ldg(qent + r);
                const unsigned row = div_m(e & ~kDupFlag);
                const unsigned row0 = __shfl_sync(kFull, row, lane & 24);       // target 0's row, same position
                uniform = uniform && !(e & kDupFlag) && row == row0;
            }
            uniform = __all_sync(kFull, uniform);
        } else {
            uniform = false;
        }
        if (uniform) {
            const int per = kUC / ic;                                        // entries per pass
            for (int r0 = 0; r0 < maxlen; r0 += per) {
                const int Lc = min(per, maxlen - r0);
                __syncwarp();
                // weight element of every (source row, target) and the source rows
                for (int r = psub; r < Lc; r += 4) {
                    const unsigned plain = (unsigned)__ldg(qent + r0 + r);
                    for (int k = 0; k < ic; ++k) edge[(r * ic + k) * kT + myq] = plain * (unsigned)ic + (unsigned)k;
                    if (myq == 0) {
                        const unsigned src = div_m(plain) * (unsigned)ic;
                        for (int k = 0; k < ic; ++k) uniq[r * ic + k] = (unsigned short)(src + k);
                    }
                }
                __syncwarp();
                dense_heads(Lc * ic, r0 == 0);
            }
            continue;
        }

        // ---- the fanned-out segments of the 8 targets, concatenated
        const int flen = len * ic;                              // lanes 0..7: edges of target `lane`
        int incl = flen;
#pragma unroll
        for (int o = 1; o < kT; o <<= 1) {
            const int y = __shfl_up_sync(kFull, incl, o);
            if (lane >= o) incl += y;
        }
        const int E_total = __shfl_sync(kFull, incl, kT - 1);
        int off[kT], st[kT];                                    // per tile row: offset in the edge list, segment start
#pragma unroll
        for (int r = 0; r < kT; ++r) {
            off[r] = __shfl_sync(kFull, incl - flen, r);
            st[r] = __shfl_sync(kFull, start, r);
        }
        unsigned pk[kT];                                        // (segment start - offset) << 3 | tile row
#pragma unroll
        for (int r = 0; r < kT; ++r) pk[r] = ((unsigned)(st[r] - off[r]) << 3) | (unsigned)r;

        // ---- general tile, kES edges at a time
        for (int e0 = 0; e0 == 0 || e0 < E_total; e0 += kES) {
            const int E = max(0, min(kES, E_total - e0));
            // ---- this chunk's edges: weight index (flagged when the target repeats in its row), source
            //      row, tile row
            int lo = INT_MAX, hi = -1;
            bool any_flag = false;
            __syncwarp();
#pragma unroll 4
            for (int x = lane; x < E; x += 32) {
                const int pe = e0 + x;
                int r;
                unsigned qe, k;
                int s0;
                if (ATT48) {
                    // ic = 1: entry address = (segment start - offset in the edge list) + pe; that difference
                    // and the tile row travel through one select chain (the offsets ascend)
                    unsigned v = pk[0];
#pragma unroll
                    for (int j = 1; j < kT; ++j) v = pe >= off[j] ? pk[j] : v;
                    r = (int)(v & 7u);
                    s0 = (int)(v >> 3);
                    qe = (unsigned)pe;
                    k = 0u;
                } else {
                    r = 0;
#pragma unroll
                    for (int j = 1; j < kT; ++j) r += (pe >= off[j]) ? 1 : 0;
                    s0 = st[0];
                    int o0 = off[0];
#pragma unroll
                    for (int j = 1; j < kT; ++j)
                        if (r == j) {
                            s0 = st[j];
                            o0 = off[j];
                        }
                    const unsigned q = (unsigned)(pe - o0);                 // position inside the fanned-out segment
                    qe = div_ic(q);                                         // entry inside the segment
                    k = q - qe * (unsigned)ic;
                }
                const unsigned e = (unsigned)__ldg(entries + s0 + (int)qe);
                const unsigned plain = e & ~kDupFlag;                       // row * m + slot
                const unsigned src = div_m(plain);
                edge[x] = (plain * (unsigned)ic + k) | (e & kDupFlag);
                const int srow = (int)(src * (unsigned)ic + k);
                ds.tok[x] = (unsigned short)srow;
                lut[x] = (unsigned short)(r << 12);                         // the slot is merged in below
                lo = min(lo, srow);
                hi = max(hi, srow);
                if (e & kDupFlag) any_flag = true;
            }
            any_flag = __any_sync(kFull, any_flag);
            int U = 0;
            if (E > 0) {
                bool unused = false;
                U = dedup_tokens(ds, slots, E, m, false, &unused, lane, lo, hi);
                for (int x = lane; x < E; x += 32) lut[x] = (unsigned short)(lut[x] | slots[x]);
            }
            __syncwarp();

            for (int g = 0; g < p.heads; ++g) {
                const T* Wh = Wg + (long long)b * p.w_batch + (long long)g * p.w_head;
                const T* Xh = Xg + (long long)b * p.x_batch + (long long)g * p.x_head;
                // ---- weights of the edges for this slab
                if (g == 0 || p.w_head != 0) {
                    if (kIsFloat) {
                        // asynchronous 4-byte copies: all of a lane's weights are in flight together with the
                        // rows staged below; both are waited for before the dense weights are filled in
#pragma unroll 4
                        for (int x = lane; x < E; x += 32) {
                            const unsigned e = edge[x];
                            if (e & kDupFlag) wbuf[x] = 0.f;
                            else cp_async4_ca(wbuf + x, Wh + e);
                        }
                    } else if (!any_flag && p.w_pairs) {
                        // 16-bit weights: copy the aligned 32-bit word that holds the element; the half is
                        // picked when the dense weights are filled in
#pragma unroll 4
                        for (int x = lane; x < E; x += 32) {
                            const uintptr_t a = reinterpret_cast<uintptr_t>(Wh + edge[x]);
                            cp_async4_ca(wbuf + x, reinterpret_cast<const void*>(a & ~uintptr_t(3)));
                        }
                    } else {
#pragma unroll 4
                        for (int x = lane; x < E; x += 32) {
                            const unsigned e = edge[x];
                            wbuf[x] = (e & kDupFlag) ? 0.f : Elem<T>::up(Wh[e]);
                        }
                    }
                    if (any_flag) {
                        // targets that occur several times in their source row: sum that row's slots in order
                        for (int x = lane; x < E; x += 32) {
                            const unsigned e = edge[x];
                            if (e & kDupFlag) {
                                const unsigned we = e & ~kDupFlag;
                                const unsigned pl = div_ic(we);
                                const unsigned k = we - pl * (unsigned)ic;
                                const unsigned row = div_m(pl);
                                const int t = t0 + (lut[x] >> 12);
                                const int64_t* irow = idx_b + (long long)row * m;
                                float w = 0.f;
#pragma unroll 1
                                for (int j = 0; j < m; ++j)
                                    if (irow[j] == t) w += Elem<T>::up(Wh[((long long)row * m + j) * ic + k]);
                                wbuf[x] = w;
                            }
                        }
                    }
                }
                float acc[2][4];
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[0][i] = acc[1][i] = 0.f;
                for (int u0 = 0; u0 < U; u0 += kUC) {
                    const int Uc = min(kUC, U - u0);
                    const int rows8 = (Uc + 7) & ~7;
                    const int rows16 = (Uc + 15) & ~15;
                    __syncwarp();
                    if (kIsFloat) {
#pragma unroll
                        for (int k = 0; k < kUC / 4; ++k) {
                            const int r = qi + 4 * k;
                            if (r < rows8) {
                                float* dst = Xs + r * kC + sw;
                                if (r < Uc) cp_async16_cg(dst, Xh + (long long)uniq[u0 + r] * x_row + ci * 4);
                                else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
                            }
                        }
                    } else {
                        const int pr = lane >> 2, pc = lane & 3;
#pragma unroll
                        for (int k = 0; k < kUC / 8; ++k) {
                            const int r = pr + 8 * k;
                            if (r < rows16) {
                                T* dst = Xraw + swz16(r, pc);
                                if (r < Uc) cp_async16_cg(dst, Xh + (long long)uniq[u0 + r] * x_row + pc * kPer);
                                else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
                            }
                        }
                    }
                    cp_async_commit();
                    // 16-bit inputs stay 16-bit unless a weight of this chunk is a sum over repeated slots
                    const bool native16 = !kIsFloat && !any_flag;
                    for (int z = lane; z < kT * kWLD / 4; z += 32)
                        reinterpret_cast<float4*>(Wd)[z] = make_float4(0.f, 0.f, 0.f, 0.f);
                    cp_async_wait<0>();
                    __syncwarp();
#pragma unroll 4
                    for (int x = lane; x < E; x += 32) {
                        const unsigned lr = lut[x];
                        const int rel = (int)(lr & 0xfffu) - u0;
                        if (rel >= 0 && rel < Uc) {
                            if (native16 && p.w_pairs) {
                                const unsigned raw = reinterpret_cast<const unsigned*>(wbuf)[x];
                                const bool high = (reinterpret_cast<uintptr_t>(Wh + edge[x]) & 2) != 0;
                                reinterpret_cast<unsigned short*>(Wd16)[(lr >> 12) * kWLD16 + rel] =
                                    (unsigned short)(high ? raw >> 16 : raw & 0xffffu);
                            } else if (native16) {
                                Wd16[(lr >> 12) * kWLD16 + rel] = Elem<T>::down(wbuf[x]);
                            } else {
                                Wd[(lr >> 12) * kWLD + rel] = wbuf[x];
                            }
                        }
                    }
                    __syncwarp();
                    if (!kIsFloat && !native16) {
#pragma unroll
                        for (int k = 0; k < kUC / 4; ++k) {
                            const int r = qi + 4 * k;
                            if (r < rows8) st4(Xs + r * kC + sw, ld4(Xraw + swz16(r, ci >> 1) + (ci & 1) * 4));
                        }
                        __syncwarp();
                    }
                    if (native16) sum_product16<T>(Xraw, Wd16, rows16 >> 4, lane, acc);
                    else sum_product_mma<kIsFloat>(sa, rows8, acc);
                }
                // D fragments -> output tile in shared memory -> 16-byte stores (added to what earlier
                // chunks of a long edge list wrote)
                float* Ot = Wd;
                const int gg = lane >> 2, tt = lane & 3;
                __syncwarp();
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    float* o = Ot + (2 * tt) * kOLD + 16 * mt + gg;
                    o[0] = acc[mt][0];
                    o[kOLD] = acc[mt][1];
                    o[8] = acc[mt][2];
                    o[kOLD + 8] = acc[mt][3];
                }
                __syncwarp();
                T* Oh = Og + (long long)b * p.o_batch + (long long)g * p.o_head;
#pragma unroll
                for (int a = 0; a < 2; ++a) {
                    const int q = 2 * qi + a;
                    if (t0 + q < n_tgt) {
                        T* dstp = Oh + (long long)(t0 + q) * o_row + ci * 4;
                        float4 v = *reinterpret_cast<const float4*>(Ot + q * kOLD + ci * 4);
                        if (e0 > 0) {
                            const float4 old = ld4(dstp);
                            v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
                        }
                        st4(dstp, v);
                    }
                }
                __syncwarp();
            }
        }
    }
}

// ----------------------------------------------------------------------------- host side
bool gather_supported(int dtype, std::initializer_list<const void*> ptrs, int n, int m, int c) {
    if (c != kC || m < 1 || m > kMmax || n < 1 || n > 65000) return false;
    if (dtype != CLUSTEN_F32 && dtype != CLUSTEN_F16 && dtype != CLUSTEN_BF16) return false;
    for (const void* p : ptrs)
        if (reinterpret_cast<uintptr_t>(p) % 16 != 0) return false;
    return true;
}

template <typename T, int MODE>
int gather_tiles_t(const char* label, const void* A, const void* X, const int64_t* idx, void* out, int b, int h,
                   int n, int m, cudaStream_t s, GatherStrides gs) {
    if (gs.x_row == 0) {                       // contiguous [b, h, n, 32]
        gs.x_batch = (long long)h * n * kC;  gs.x_head = (long long)n * kC;  gs.x_row = kC;
    }
    if (gs.y_row == 0) {
        gs.y_batch = (long long)h * n * kC;  gs.y_head = (long long)n * kC;  gs.y_row = kC;
    }
    const int tiles = (n + kT - 1) / kT;
    if ((long long)b * tiles > 0x7fffffffLL) return CLUSTEN_ERR_SHAPE;
    const size_t smem = size_t(kWarps) * WarpSmem<T, MODE>::kTotal;
    auto kernel = m == kMmax ? gather_tiles_kernel<T, MODE, true> : gather_tiles_kernel<T, MODE, false>;
    // one resident wave of CTAs; every warp strides over the (batch, tile) pairs
    const int per_sm = resident_ctas(reinterpret_cast<const void*>(kernel), 32 * kWarps, smem);
    if (per_sm < 0) return per_sm;
    long long grid = (long long)sm_count() * per_sm;
    const long long need = ((long long)b * tiles + kWarps - 1) / kWarps;
    if (grid > need) grid = need;
    ScopedKernelTimer timer(label, s);
    kernel<<<(int)grid, 32 * kWarps, smem, s>>>((const T*)A, (const T*)X, idx, (T*)out, b, h, n, m, tiles, gs);
    note_launch();
    return check_launch();
}

// magic numbers for x / d with x < 2^31: q = (umulhi(magic, x) + x) >> shift
void div_magic(unsigned d, unsigned* magic, unsigned* shift) {
    unsigned l = 0;
    while ((1ull << l) < d) ++l;
    *magic = (unsigned)(((1ull << 32) * ((1ull << l) - d)) / d + 1);
    *shift = l;
}

template <typename T>
int scatter_tiles_t(const char* label, ScatterParams p, cudaStream_t s) {
    p.tiles = (p.n_tgt + kT - 1) / kT;
    if ((long long)p.batch * p.tiles > 0x7fffffffLL) return CLUSTEN_ERR_SHAPE;
    div_magic((unsigned)p.m, &p.m_magic, &p.m_shift);
    div_magic((unsigned)p.ic, &p.ic_magic, &p.ic_shift);
    // reading the 32-bit word around a 16-bit element stays inside W when W starts on a 4-byte boundary
    // and holds an even number of elements
    p.w_pairs = reinterpret_cast<uintptr_t>(p.W) % 4 == 0 && p.w_batch % 2 == 0;
    const size_t smem = size_t(kWarps) * ScatterSmem<T>::kTotal;
    auto kernel = (p.m == 48 && p.ic == 1) ? scatter_tiles_kernel<T, true> : scatter_tiles_kernel<T, false>;
    const int per_sm = resident_ctas(reinterpret_cast<const void*>(kernel), 32 * kWarps, smem);
    if (per_sm < 0) return per_sm;
    long long grid = (long long)sm_count() * per_sm;
    const long long need = ((long long)p.batch * p.tiles + kWarps - 1) / kWarps;
    if (grid > need) grid = need;
    ScopedKernelTimer timer(label, s);
    kernel<<<(int)grid, 32 * kWarps, smem, s>>>(p);
    note_launch();
    return check_launch();
}

int scatter_dispatch(const char* label, int dtype, const ScatterParams& p, cudaStream_t s) {
    switch (dtype) {
        case CLUSTEN_F32: return scatter_tiles_t<float>(label, p, s);
        case CLUSTEN_F16: return scatter_tiles_t<__half>(label, p, s);
        case CLUSTEN_BF16: return scatter_tiles_t<__nv_bfloat16>(label, p, s);
        default: return CLUSTEN_ERR_DTYPE;
    }
}

}  // namespace

bool tiled_sum_supported(int dtype, const void* W, const void* X, const void* out, int n, int m, int c) {
    return gather_supported(dtype, {W, X, out}, n, m, c);
}
int launch_tiled_sum(const char* label, int dtype, const void* W, const void* X, const int64_t* idx, void* out,
                     int b, int h, int n, int m, cudaStream_t s, const GatherStrides& gs) {
    switch (dtype) {
        case CLUSTEN_F32: return gather_tiles_t<float, 0>(label, W, X, idx, out, b, h, n, m, s, gs);
        case CLUSTEN_F16: return gather_tiles_t<__half, 0>(label, W, X, idx, out, b, h, n, m, s, gs);
        case CLUSTEN_BF16: return gather_tiles_t<__nv_bfloat16, 0>(label, W, X, idx, out, b, h, n, m, s, gs);
        default: return CLUSTEN_ERR_DTYPE;
    }
}

bool tiled_dot_supported(int dtype, const void* Y, const void* X, const void* out, int n, int m, int c) {
    return gather_supported(dtype, {Y, X, out}, n, m, c);
}
int launch_tiled_dot(const char* label, int dtype, const void* X, const void* Y, const int64_t* idx, void* out,
                     int b, int h, int n, int m, cudaStream_t s, const GatherStrides& gs) {
    switch (dtype) {
        case CLUSTEN_F32: return gather_tiles_t<float, 1>(label, Y, X, idx, out, b, h, n, m, s, gs);
        case CLUSTEN_F16: return gather_tiles_t<__half, 1>(label, Y, X, idx, out, b, h, n, m, s, gs);
        case CLUSTEN_BF16: return gather_tiles_t<__nv_bfloat16, 1>(label, Y, X, idx, out, b, h, n, m, s, gs);
        default: return CLUSTEN_ERR_DTYPE;
    }
}

}  // namespace clusten

namespace clusten {

bool tiled_scatter_supported(int dtype, const void* W, const void* X, const void* out, int n, int m, int c) {
    return gather_supported(dtype, {X, out}, n, 1, c) && m >= 1 && reinterpret_cast<uintptr_t>(W) % 4 == 0;
}
int launch_tiled_scatter(const char* label, int dtype, const void* W, const void* X, const int64_t* idx,
                         const InverseView& inv, void* out, int b, int h, int n, int m, cudaStream_t s) {
    ScatterParams p{};
    p.W = W;  p.w_batch = (long long)h * n * m;  p.w_head = (long long)n * m;
    p.X = X;  p.x_batch = (long long)h * n * kC; p.x_head = (long long)n * kC;  p.x_row = kC;
    p.out = out;  p.o_batch = p.x_batch;  p.o_head = p.x_head;  p.o_row = kC;
    p.idx = idx;  p.idx_rows = n;  p.m = m;  p.inv = inv;  p.n_tgt = n;
    p.ic = 1;  p.heads = h;  p.batch = b;
    // tiles whose structure the inverse build recorded go to the lean kernel, the others to the general one
    const bool lean = reinterpret_cast<uintptr_t>(W) % 16 == 0;
    if (lean) {
        const int st = launch_struct_scatter(label, dtype, W, X, inv, out, b, h, n, m, s);
        if (st != CLUSTEN_OK) return st;
    }
    p.skip_flagged = lean ? 1 : 0;
    return scatter_dispatch(label, dtype, p, s);
}

// WF: d_feat[b, t, :] over c channels in slabs of 32; rows of X are d_feat_new[b, i, k, :]
bool tiled_wf_scatter_supported(int dtype, const void* W, const void* X, const void* out, int n_out, int n, int m,
                                int ic, int c) {
    if (dtype != CLUSTEN_F32 && dtype != CLUSTEN_F16 && dtype != CLUSTEN_BF16) return false;
    if (c % kC != 0 || ic < 1 || ic > 16 || m < 1 || n < 1 || (long long)n_out * ic > 65000) return false;
    return reinterpret_cast<uintptr_t>(X) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0 &&
           reinterpret_cast<uintptr_t>(W) % 4 == 0;
}
int launch_tiled_wf_scatter(const char* label, int dtype, const void* W, const void* X, const int64_t* idx,
                            const InverseView& inv, void* out, int b, int n_out, int n, int m, int ic, int c,
                            cudaStream_t s) {
    ScatterParams p{};
    p.W = W;  p.w_batch = (long long)n_out * m * ic;  p.w_head = 0;
    p.X = X;  p.x_batch = (long long)n_out * ic * c;  p.x_head = kC;  p.x_row = c;
    p.out = out;  p.o_batch = (long long)n * c;  p.o_head = kC;  p.o_row = c;
    p.idx = idx;  p.idx_rows = n_out;  p.m = m;  p.inv = inv;  p.n_tgt = n;
    p.ic = ic;  p.heads = c / kC;  p.batch = b;
    return scatter_dispatch(label, dtype, p, s);
}

}  // namespace clusten
