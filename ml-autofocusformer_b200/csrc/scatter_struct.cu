// Scatter-side gradients of QK / AV (d_key, d_value) on STRUCTURED tiles of the inverse index:
//
//   out[b, h, t, :] = sum over entries (i, j) of target t:  W[b, h, i, j] * X[b, h, i, :]        (head_dim 32)
//
// The inverse build marks the tiles of 8 consecutive targets whose segments have one of the two
// shapes AutoFocusFormer's neighbour tables produce (common.cuh, kTileRuns / kTileClusters).  For such
// a tile nothing has to be analysed per edge:
//
//   runs      the 8 targets are named by the same L rows, target q at slot j0 + q.  The source rows are
//             the staged rows, and the 8 weights of a row are 8 neighbouring elements of W: one or
//             two 16-byte copies per row fill the dense [L x 8] weight tile.
//   clusters  every segment is made of whole clusters (8 rows 8c .. 8c+7 at one slot).  The (cluster,
//             slot) pairs of the tile, at most 96, are de-duplicated by cluster (about ten distinct
//             ones); each distinct cluster is staged as 8 consecutive rows (one contiguous kilobyte in
//             fp32) and a pair contributes one column of 8 weights.
//
// Either way the product out[8 x 32] = Wd[8 x K] * X[K x 32] runs on the tensor cores, 48 staged rows
// at a time (mma.sync: TF32 in three passes for FP32 inputs, m16n8k16 for FP16 / BF16), with a fixed
// summation order.  Every warp works alone on one tile and all heads.  Tiles that are not marked are
// left to scatter_tiles_kernel (tiled_fwd.cu).  The reference adds every (row, slot, channel) term
// with atomicAdd (clusten/src/clustenqk_cuda_kernel.cu:117-127, clustenav_cuda_kernel.cu:113-123).
#include "tile_core.cuh"

namespace clusten {
namespace {

constexpr int kSR = 32;                  // staged rows per stage (4 clusters)
constexpr int kPairs = kStructMaxPairs;  // (cluster, slot) pairs of a clusters tile; entries kept of a runs tile

// Per-warp shared memory.  One buffer of rows and weights: a second one, filled while the first is multiplied,
// measured slower than the extra resident warps that its 5 KB per warp pay for (7 CTAs per SM instead of 4).
template <typename T> struct StructSmem {
    static constexpr bool kIsFloat = std::is_same<T, float>::value;
    static constexpr int kX = kSR * kC * (int)sizeof(T);      // staged rows, one buffer; de-duplication scratch before that
    static constexpr int kW = kSR * kT * (int)sizeof(T);      // dense weights [staged row][target], one buffer
    static constexpr int kOut = kT * kOLD * 4;                // output tile
    static constexpr int kCode = kPairs * 4;                  // clusters: offset of a pair's first weight;  runs: the entries
    static constexpr int kSlotq = kPairs * 2;                 // clusters: slot of the pair's cluster | target << 12
    static constexpr int kUniq = kPairs * 2;                  // clusters: slot -> cluster
    static constexpr int kJmap = kPairs * kT;                 // clusters: [slot][target] -> neighbour slot j, 0xff = not named
    static constexpr int kTotal = kX + kW + kOut + kCode + kSlotq + kUniq + kJmap;
};
static_assert(kPairs * 2 + kBMW * 4 + kBMW * 2 + 64 <= kSR * kC * 2, "de-duplication scratch must fit in the row buffers");
static_assert(StructSmem<float>::kTotal % 128 == 0 && StructSmem<__half>::kTotal % 128 == 0, "warps stay 128-byte aligned");

struct StructParams {
    const void* W;      // [batch][heads][n][m]
    const void* X;      // [batch][heads][n][32]
    void* out;          // [batch][heads][n][32]
    InverseView inv;
    int batch, heads, n, m, tiles;
    unsigned m_magic, m_shift;
};

__device__ __forceinline__ unsigned struct_div(unsigned x, unsigned magic, unsigned shift) {
    return (__umulhi(magic, x) + x) >> shift;
}

// D[ch][q] += sum_u Xs[u][ch] * Ws[u][q] over 8 * ksteps staged rows, FP32 inputs as three TF32 passes.
// Xs rows are [32] floats with 16-byte chunk c of row r at c ^ ((r & 3) << 1); Ws is [row][8].
struct StructAddr {
    unsigned w;          // &Ws[t][g]
    unsigned x[2][2];    // &Xs[t][16 mt + 8 h + g]
};
__device__ __forceinline__ StructAddr make_struct_addr(const float* Ws, const float* Xs, int lane) {
    const int g = lane >> 2, t = lane & 3;
    StructAddr a;
    a.w = smem_u32(Ws + t * kT + g);
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int c = 16 * mt + 8 * h + g;
            a.x[mt][h] = smem_u32(Xs + t * kC + ((((c >> 2) ^ (t << 1)) << 2) + (c & 3)));
        }
    return a;
}
template <int KS>
__device__ __forceinline__ void struct_load(const StructAddr& sa, float (&b)[2], float (&a)[2][4]) {
    asm volatile("ld.shared.f32 %0, [%1+%2];\n" : "=f"(b[0]) : "r"(sa.w), "n"(KS * 8 * kT * 4));
    asm volatile("ld.shared.f32 %0, [%1+%2];\n" : "=f"(b[1]) : "r"(sa.w), "n"((KS * 8 + 4) * kT * 4));
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
        asm volatile("ld.shared.f32 %0, [%1+%2];\n" : "=f"(a[mt][0]) : "r"(sa.x[mt][0]), "n"(KS * 8 * kC * 4));
        asm volatile("ld.shared.f32 %0, [%1+%2];\n" : "=f"(a[mt][1]) : "r"(sa.x[mt][1]), "n"(KS * 8 * kC * 4));
        asm volatile("ld.shared.f32 %0, [%1+%2];\n" : "=f"(a[mt][2]) : "r"(sa.x[mt][0]), "n"((KS * 8 + 4) * kC * 4));
        asm volatile("ld.shared.f32 %0, [%1+%2];\n" : "=f"(a[mt][3]) : "r"(sa.x[mt][1]), "n"((KS * 8 + 4) * kC * 4));
    }
}
template <int KS>
__device__ __forceinline__ void struct_steps(const StructAddr& sa, int ksteps, float (&acc)[2][4]) {
    if constexpr (KS < kSR / 8) {
        if (KS < ksteps) {
            float b[2], a[2][4];
            struct_load<KS>(sa, b, a);
            mma_pair<true>(acc, a, b);
            struct_steps<KS + 1>(sa, ksteps, acc);
        }
    }
}

// 16-bit inputs: Xraw rows [32] elements, 16-byte chunk c of row r at c ^ ((r >> 1) & 3) (swz16);
// Ws16 is [row][8].  A = X^T through ldmatrix.trans, B = Ws16 through ldmatrix.trans (8 x 8 blocks of
// [row][target] give the (k = row pair, n = target) fragment).
template <typename T>
__device__ __forceinline__ void struct_product16(const T* Xraw, const T* Ws16, int ksteps16, int lane, float (&acc)[2][4]) {
    const int mi = lane >> 3, rr = lane & 7;
    unsigned xa[2];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) xa[mt] = smem_u32(Xraw + swz16((mi >> 1) * 8 + rr, 2 * mt + (mi & 1)));
    // lanes 0..15 address rows 0..15 of the step (matrix 0: rows 0..7, matrix 1: rows 8..15)
    const unsigned wa = smem_u32(Ws16 + (lane & 15) * kT);
#pragma unroll
    for (int ks = 0; ks < kSR / 16; ++ks) {
        if (ks < ksteps16) {
            unsigned b[2];
            asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n"
                         : "=r"(b[0]), "=r"(b[1]) : "r"(wa + ks * 16 * kT * 2));
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
                unsigned a[4];
                ldsm_x4_trans(a, xa[mt] + ks * 16 * kC * 2);
                mma16(acc[mt], a, b, static_cast<const T*>(nullptr));
            }
        }
    }
}

template <typename T, bool M48>
__global__ void __launch_bounds__(32 * kWarps, sizeof(T) == 4 ? 7 : 6)
scatter_struct_kernel(const StructParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    using WS = StructSmem<T>;
    constexpr bool kIsFloat = WS::kIsFloat;
    constexpr int kPer = 16 / (int)sizeof(T);           // elements per 16-byte piece
    constexpr int kLanesPerRow = kC / kPer;             // 8 (fp32) or 4 (16-bit)
    constexpr int kRowsPerPass = 32 / kLanesPerRow;     // 4 or 8
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned char* base = smem_raw + size_t(warp) * WS::kTotal;
    T* Xs = reinterpret_cast<T*>(base);                                         // [kSR][32]
    T* Ws = reinterpret_cast<T*>(base + WS::kX);                                // [kSR][8]
    float* Ot = reinterpret_cast<float*>(base + WS::kX + WS::kW);
    unsigned* code = reinterpret_cast<unsigned*>(Ot + kT * kOLD);
    unsigned short* slotq = reinterpret_cast<unsigned short*>(code + kPairs);
    unsigned short* uniq = slotq + kPairs;
    unsigned char* jmap = reinterpret_cast<unsigned char*>(uniq + kPairs);
    DedupScratch ds;
    ds.tok = reinterpret_cast<unsigned short*>(base);
    ds.bm = reinterpret_cast<unsigned*>(base + kPairs * 2);
    ds.pre = reinterpret_cast<unsigned short*>(ds.bm + kBMW);
    ds.rowbm = reinterpret_cast<unsigned*>(ds.pre + kBMW);
    ds.uniq = uniq;

    const int m = M48 ? 48 : p.m, n = p.n, heads = p.heads;
    auto div_m = [&](unsigned x) { return M48 ? x / 48u : struct_div(x, p.m_magic, p.m_shift); };
    const T* Wg = static_cast<const T*>(p.W);
    const T* Xg = static_cast<const T*>(p.X);
    T* Og = static_cast<T*>(p.out);
    const int pr = lane / kLanesPerRow, pc = lane % kLanesPerRow;       // staging: row within a pass, 16-byte piece
    // element offset of this lane's piece of staged row r inside a row buffer (chunk swizzle of the products)
    auto xoff = [&](int r) { return kIsFloat ? r * kC + ((pc ^ ((r & 3) << 1)) << 2) : swz16(r, pc); };
    StructAddr sa0{};
    if (kIsFloat) sa0 = make_struct_addr(reinterpret_cast<const float*>(Ws), reinterpret_cast<const float*>(Xs), lane);

    const unsigned total = (unsigned)p.batch * (unsigned)p.tiles;
    const unsigned nwarps = gridDim.x * kWarps;
    // kind, and (lanes 0..7) segment length and start of the targets of a task's tile
    auto load_meta = [&](unsigned task, int& kind, int& len, int& start) {
        kind = kTileGeneral;
        len = 0;
        start = 0;
        if (task < total) {
            const int b = (int)(task / (unsigned)p.tiles);
            const int tile = (int)(task - (unsigned)b * (unsigned)p.tiles);
            kind = __ldg(p.inv.tileflag + (long long)b * (1 + p.inv.ntiles) + 1 + tile);
            const int t = tile * kT + lane;
            if (lane < kT && t < n) {
                len = __ldg(p.inv.seglen + (long long)b * n + t);
                start = __ldg(p.inv.rowptr + (long long)b * (n + 1) + t);
            }
        }
    };
    int next_kind, next_len, next_start;
    load_meta(blockIdx.x * kWarps + warp, next_kind, next_len, next_start);
    for (unsigned task = blockIdx.x * kWarps + warp; task < total; task += nwarps) {
        const int kind = next_kind, len = next_len, start = next_start;
        load_meta(task + nwarps, next_kind, next_len, next_start);      // in flight while this tile is worked on
        if (kind == kTileGeneral) continue;
        const int b = (int)(task / (unsigned)p.tiles);
        const int t0 = (int)(task - (unsigned)b * (unsigned)p.tiles) * kT;
        const int* entries = p.inv.entries + (long long)b * n * m;
        __syncwarp();

        int L = 0, UC = 0;                 // runs: rows of the tile;  clusters: pairs and distinct clusters
        int start0 = 0;
        if (kind == kTileRuns) {
            L = __shfl_sync(kFull, len, 0);
            start0 = __shfl_sync(kFull, start, 0);
            for (int x = lane; x < min(L, kPairs); x += 32) code[x] = (unsigned)__ldg(entries + start0 + x);
            __syncwarp();
        } else {
            // ---- the tile's (cluster, slot) pairs: first entry of every group of 8
            const int pairs = len >> 3;
            int incl = pairs;
#pragma unroll
            for (int o = 1; o < kT; o <<= 1) {
                const int y = __shfl_up_sync(kFull, incl, o);
                if (lane >= o) incl += y;
            }
            const int CE = __shfl_sync(kFull, incl, kT - 1);
            int off[kT], st[kT];
#pragma unroll
            for (int j = 0; j < kT; ++j) {
                off[j] = __shfl_sync(kFull, incl - pairs, j);
                st[j] = __shfl_sync(kFull, start, j);
            }
            int lo = INT_MAX, hi = -1;
            unsigned myq[(kPairs + 31) / 32];
#pragma unroll
            for (int i = 0; i < (kPairs + 31) / 32; ++i) {
                const int x = lane + 32 * i;
                int q = 0;
#pragma unroll
                for (int j = 1; j < kT; ++j) q += x >= off[j] ? 1 : 0;
                int o = off[0], s0 = st[0];
#pragma unroll
                for (int j = 1; j < kT; ++j)
                    if (q == j) {
                        o = off[j];
                        s0 = st[j];
                    }
                myq[i] = (unsigned)q;
                if (x < CE) {
                    const unsigned e = (unsigned)__ldg(entries + s0 + 8 * (x - o));
                    const int c = (int)(div_m(e) >> 3);
                    code[x] = e;
                    ds.tok[x] = (unsigned short)c;
                    lo = min(lo, c);
                    hi = max(hi, c);
                }
            }
            bool unused = false;
            UC = CE > 0 ? dedup_tokens(ds, slotq, CE, m, false, &unused, lane, lo, hi) : 0;
            // per distinct cluster: the slot at which it names each of the 8 targets (a flagged tile has at
            // most one), 0xff where it does not
            for (int z = lane; z < UC * kT / 4; z += 32) reinterpret_cast<unsigned*>(jmap)[z] = 0xffffffffu;
            __syncwarp();
#pragma unroll
            for (int i = 0; i < (kPairs + 31) / 32; ++i) {
                const int x = lane + 32 * i;
                if (x < CE) {
                    const unsigned e = code[x];
                    jmap[(int)slotq[x] * kT + (int)myq[i]] = (unsigned char)(e - div_m(e) * (unsigned)m);
                }
            }
            L = CE;
            __syncwarp();
        }

        const int nstages = kind == kTileRuns ? (L + kSR - 1) / kSR : (UC + 3) / 4;
        const int units = heads * nstages;
        // rows of stage s, and rounded up to what the product consumes
        auto stage_rows = [&](int s) { return kind == kTileRuns ? min(kSR, L - s * kSR) : 8 * min(4, UC - 4 * s); };
        auto padded = [&](int rows) { return kIsFloat ? ((rows + 7) & ~7) : ((rows + 15) & ~15); };
        // clusters tiles: lane l copies piece l of a cluster's 8 contiguous rows (fp32: two pieces, rows l / 8 and
        // 4 + l / 8; 16-bit: row l / 4) and fills weight (row l % 8, targets l / 8 and 4 + l / 8)
        const int wr = lane & 7, wq = lane >> 3;
        const int xrow = kIsFloat ? (lane >> 3) : (lane >> 2);

        // ---- loads of unit (head g, stage s); the weights of a clusters tile come back in wv (plain loads, in
        //      flight together with the asynchronous row copies) and are stored by the caller
        auto issue = [&](int g, int s, T (&wv)[8]) {
            const long long bh = (long long)b * heads + g;
            const T* Wh = Wg + bh * n * m;
            const T* Xh = Xg + bh * n * kC;
            T* Xb = Xs;
            T* Wb = Ws;
            const int rows = stage_rows(s), rows_pad = padded(rows);
            if (kind == kTileRuns) {
                const int k0 = s * kSR;
                auto entry = [&](int r) {
                    return k0 + r < kPairs ? code[k0 + r] : (unsigned)__ldg(entries + start0 + k0 + r);
                };
#pragma unroll
                for (int k = 0; k < kSR / kRowsPerPass; ++k) {
                    const int r = pr + kRowsPerPass * k;
                    if (r < rows_pad) {
                        T* dst = Xb + xoff(r);
                        if (r < rows) cp_async16_cg(dst, Xh + (long long)div_m(entry(r)) * kC + pc * kPer);
                        else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
                constexpr int kPieces = kT / kPer;      // 16-byte pieces per row of 8 weights: 2 or 1
#pragma unroll
                for (int k = 0; k < kSR * kPieces / 32; ++k) {
                    const int z = lane + 32 * k;
                    const int r = z / kPieces, piece = z % kPieces;
                    if (r < rows_pad) {
                        T* dst = Wb + r * kT + piece * kPer;
                        if (r < rows) cp_async16_ca(dst, Wh + entry(r) + piece * kPer);
                        else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int u = 4 * s + i;
                    if (u < UC) {
                        const int c8 = (int)uniq[u] * 8;                    // first row of the cluster
                        const T* xsrc = Xh + (long long)c8 * kC + lane * kPer;
                        if (kIsFloat) {
                            cp_async16_cg(Xb + xoff(8 * i + xrow), xsrc);
                            cp_async16_cg(Xb + xoff(8 * i + 4 + xrow), xsrc + 4 * kC);
                        } else {
                            cp_async16_cg(Xb + xoff(8 * i + xrow), xsrc);
                        }
                        const T* wsrc = Wh + (long long)(c8 + wr) * m;
#pragma unroll
                        for (int h2 = 0; h2 < 2; ++h2) {
                            const int q = wq + 4 * h2;
                            const unsigned j = jmap[u * kT + q];
                            wv[2 * i + h2] = j != 0xffu ? wsrc[j] : Elem<T>::down(0.f);
                        }
                    } else if (8 * i < rows_pad) {
                        // 16-bit products run over multiples of 16 rows: an empty cluster slot is zero
                        *reinterpret_cast<float4*>(Xb + xoff(8 * i + xrow)) = make_float4(0.f, 0.f, 0.f, 0.f);
                        wv[2 * i] = wv[2 * i + 1] = Elem<T>::down(0.f);
                    }
                }
            }
            cp_async_commit();
        };

        float acc[2][4];
        int g = 0, st = 0;
        for (int u = 0; u < units; ++u) {
            int ng = g, ns = st + 1;
            if (ns == nstages) {
                ns = 0;
                ++ng;
            }
            T wcur[8];
            issue(g, st, wcur);
            cp_async_wait<0>();
            const int rows_pad = padded(stage_rows(st));
            if (kind == kTileClusters) {
                T* Wb = Ws;
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (8 * i < rows_pad) {
                        Wb[(8 * i + wr) * kT + wq] = wcur[2 * i];
                        Wb[(8 * i + wr) * kT + wq + 4] = wcur[2 * i + 1];
                    }
            }
            __syncwarp();
            if (st == 0) {
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[0][i] = acc[1][i] = 0.f;
            }
            if (kIsFloat) struct_steps<0>(sa0, rows_pad >> 3, acc);
            else struct_product16<T>(Xs, Ws, rows_pad >> 4, lane, acc);
            __syncwarp();                                  // the buffers are refilled by the next issue
            if (st == nstages - 1) {
                // ---- D fragments -> output tile -> 16-byte stores
                const int gg = lane >> 2, tt = lane & 3;
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    float* o = Ot + (2 * tt) * kOLD + 16 * mt + gg;
                    o[0] = acc[mt][0];
                    o[kOLD] = acc[mt][1];
                    o[8] = acc[mt][2];
                    o[kOLD + 8] = acc[mt][3];
                }
                __syncwarp();
                const int qi = lane >> 3, ci = lane & 7;
                T* Oh = Og + ((long long)b * heads + g) * n * kC;
#pragma unroll
                for (int a = 0; a < 2; ++a) {
                    const int q = 2 * qi + a;
                    st4(Oh + (long long)(t0 + q) * kC + ci * 4, *reinterpret_cast<const float4*>(Ot + q * kOLD + ci * 4));
                }
                __syncwarp();
            }
            g = ng;
            st = ns;
        }
        if (units == 0 || nstages == 0) {
            // a tile nobody names: zeros
            for (int g = 0; g < heads; ++g) {
                T* Oh = Og + ((long long)b * heads + g) * n * kC;
                const int qi = lane >> 3, ci = lane & 7;
#pragma unroll
                for (int a = 0; a < 2; ++a) st4(Oh + (long long)(t0 + 2 * qi + a) * kC + ci * 4, make_float4(0.f, 0.f, 0.f, 0.f));
            }
        }
    }
}

template <typename T>
int scatter_struct_t(const char* label, StructParams p, cudaStream_t s) {
    const size_t smem = size_t(kWarps) * StructSmem<T>::kTotal;
    auto kernel = p.m == 48 ? scatter_struct_kernel<T, true> : scatter_struct_kernel<T, false>;
    const int per_sm = resident_ctas(reinterpret_cast<const void*>(kernel), 32 * kWarps, smem);
    if (per_sm < 0) return per_sm;
    long long grid = (long long)sm_count() * per_sm;
    const long long need = ((long long)p.batch * p.tiles + kWarps - 1) / kWarps;
    if (grid > need) grid = need;
    ScopedKernelTimer timer(split_timing_labels() ? "scatter_struct" : label, s);
    kernel<<<(int)grid, 32 * kWarps, smem, s>>>(p);
    note_launch();
    return check_launch();
}

}  // namespace

// Structured tiles of d_key / d_value; the other tiles are scatter_tiles_kernel's (launch_tiled_scatter).
int launch_struct_scatter(const char* label, int dtype, const void* W, const void* X, const InverseView& inv, void* out,
                          int b, int h, int n, int m, cudaStream_t s) {
    StructParams p{};
    p.W = W;  p.X = X;  p.out = out;  p.inv = inv;
    p.batch = b;  p.heads = h;  p.n = n;  p.m = m;  p.tiles = (n + kT - 1) / kT;
    if ((long long)b * p.tiles > 0x7fffffffLL) return CLUSTEN_ERR_SHAPE;
    {
        unsigned l = 0;
        while ((1ull << l) < (unsigned)m) ++l;
        p.m_magic = (unsigned)(((1ull << 32) * ((1ull << l) - (unsigned)m)) / (unsigned)m + 1);
        p.m_shift = l;
    }
    switch (dtype) {
        case CLUSTEN_F32: return scatter_struct_t<float>(label, p, s);
        case CLUSTEN_F16: return scatter_struct_t<__half>(label, p, s);
        case CLUSTEN_BF16: return scatter_struct_t<__nv_bfloat16>(label, p, s);
        default: return CLUSTEN_ERR_DTYPE;
    }
}

}  // namespace clusten
