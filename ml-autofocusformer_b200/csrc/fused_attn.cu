// Fused local attention (forward): the chain that surrounds CLUSTENQK and CLUSTENAV in the model,
//
//   attn = query x gathered keys  (+ position bias)  (+ mask)  (| blank-token logit)  -> softmax
//   out  = attn x gathered values (+ blank probability x blank value)
//
// (models/aff_transformer.py:117-155 of the reference: QK :120, bias :129-134, mask :136-137, blank token
// :140-141, softmax :142, AV :154, blank value :147,155), in one kernel.  The [b, h, n, m] attention tensor
// never reaches HBM and the neighbour indices are read once instead of twice.  The separate operators stay the
// contract of the package; this entry point is an opt-in for inference.
//
// Structure: the tile front end of the gather kernels (tiled_fwd.cu) -- a warp per tile of 8 rows, the
// tile's int64 indices read once, identical rows or a bitmap de-duplication -- and then per head three
// phases on the same shared-memory tiles: scores (stage the distinct KEY rows 48 at a time, m16n8k8 /
// m16n8k16 products, scores gathered into a [8][m] logit tile), softmax (four lanes per row, bias / mask /
// blank logit added on the way, probabilities written back in place), output (stage the distinct VALUE rows,
// dense probabilities by slot, products accumulated in registers).
#include "tile_core.cuh"

namespace clusten {
namespace {

template <typename T> struct FusedSmem {
    static constexpr bool kIsFloat = std::is_same<T, float>::value;
    static constexpr int kX = kUC * kC * (int)sizeof(T);      // staged rows (keys, then values); index landing area
    static constexpr int kYs = kT * kYLD * 4;                 // fp32: the tile's query rows
    static constexpr int kSb = kT * kWLD * 4;                 // scores of a round, by slot
    static constexpr int kP = kT * kWLD * 4;                  // logits, then probabilities, [row][neighbour]
    static constexpr int kWd = kT * kWLD * 4;                 // dense probabilities of a round, by slot (16-bit: [8][kWLD16])
    static constexpr int kLut = kE * 2;
    static constexpr int kTotal = kX + kYs + kSb + kP + kWd + 2 * kLut;
};
static_assert(kE * 8 + kE * 2 <= kUC * kC * 2 + kT * kYLD * 4 + kT * kWLD * 4, "indices and token scratch fit in front of the probability tile");
static_assert(kBMW * 4 + kBMW * 2 + (kE / 32) * 4 <= 2 * kT * kWLD * 4, "bitmap scratch fits in the probability and weight tiles");

struct FusedParams {
    const void* q;  const void* k;  const void* v;   // [b, h, n, 32] (k, v through strides)
    const int64_t* idx;                              // [b, n, m]
    const void* bias;                                // [b, h, n, m] or nullptr
    const void* table;  const int64_t* pe_idx;  int table_rows;   // [rows, h], [b, n, m] or nullptr
    const int64_t* mask;                             // [b, n, m] (1 = valid) or nullptr
    const void* blank_k;  const void* blank_v;       // [h, 32] or nullptr
    void* out;                                       // [b, h, n, 32]
    int batch, heads, n, m, tiles;
    GatherStrides gs;                                // x: keys AND values (same strides), y: queries
    int bias_aligned;                                // bias starts on a 16-byte boundary and so does every [n, m] slab
};

template <typename T, bool M48>
__global__ void __launch_bounds__(32 * kWarps, sizeof(T) == 2 ? 5 : 4)     // 16-bit: 43 KB per CTA, five fit
fused_attention_kernel(const FusedParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    using WS = FusedSmem<T>;
    constexpr bool kIsFloat = WS::kIsFloat;
    constexpr int kPer = 16 / (int)sizeof(T);
    const int m = M48 ? kMmax : p.m, n = p.n, heads = p.heads;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int qi = lane >> 3, ci = lane & 7;
    unsigned char* base = smem_raw + size_t(warp) * WS::kTotal;
    float* Xs = reinterpret_cast<float*>(base);               // fp32 rows
    T* Xraw = reinterpret_cast<T*>(base);                     // 16-bit rows (same place)
    float* Ys = reinterpret_cast<float*>(base + WS::kX);
    float* Sb = Ys + kT * kYLD;
    float* P = Sb + kT * kWLD;
    float* Wd = P + kT * kWLD;
    T* Wd16 = reinterpret_cast<T*>(Wd);
    unsigned short* lut = reinterpret_cast<unsigned short*>(Wd + kT * kWLD);
    unsigned short* uniq = lut + kE;
    long long* ring = reinterpret_cast<long long*>(base);     // [8][m] indices, in front of everything
    DedupScratch ds;
    ds.tok = reinterpret_cast<unsigned short*>(base + kE * 8);
    ds.uniq = uniq;
    ds.bm = reinterpret_cast<unsigned*>(P);
    ds.pre = reinterpret_cast<unsigned short*>(ds.bm + kBMW);
    ds.rowbm = reinterpret_cast<unsigned*>(ds.pre + kBMW);
    int* tok_s = reinterpret_cast<int*>(uniq);                // identical rows: source row of slot r

    const SumAddr sa = make_sum_addr(Wd, Xs, lane);
    const SumAddr sa_p = make_sum_addr(P, Xs, lane);            // identical rows: the probability tile is the weight matrix
    const DotAddr da = make_dot_addr(Ys, Xs, Sb, lane);
    const DotAddr da_p = make_dot_addr(Ys, Xs, P, lane);        // identical rows: slot = neighbour, scores land in P
    const int E = kT * m;
    const int col0 = (2 * lane) % m, col_step = 64 % m;
    unsigned long long qpack = 0ull;                          // 3 bits per edge of this lane: its row
#pragma unroll
    for (int k = 0; k < kEPL; ++k) qpack |= (unsigned long long)(((lane + 32 * k) / m) & 7) << (3 * k);
    const T* Qg = static_cast<const T*>(p.q);
    const T* Kg = static_cast<const T*>(p.k);
    const T* Vg = static_cast<const T*>(p.v);
    T* Og = static_cast<T*>(p.out);
    const int x_row = (int)p.gs.x_row;
    const int srow = lane >> 2, part = lane & 3;              // softmax: 4 lanes per row

    // stage the rows of slots u0 .. u0 + Uc of X (keys or values) with the swizzle of the product that follows:
    // dot = true: chunk ^ (row & 7), false: chunk ^ ((row & 3) << 1); 16-bit rows always swz16
    auto stage = [&](const T* Xh, int u0, int Uc, bool identical, bool dot) {
        if (kIsFloat) {
            const int rows8 = (Uc + 7) & ~7;
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
                    const int sw = dot ? ((ci ^ (r & 7)) << 2) : ((ci ^ ((r & 3) << 1)) << 2);
                    float* dst = Xs + r * kC + sw;
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
        cp_async_commit();
    };

    const unsigned total = (unsigned)p.batch * (unsigned)p.tiles;
    const unsigned nwarps = gridDim.x * kWarps;
    for (unsigned task = blockIdx.x * kWarps + warp; task < total; task += nwarps) {
        const int b = (int)(task / (unsigned)p.tiles);
        const int i0 = (int)(task - (unsigned)b * (unsigned)p.tiles) * kT;
        const bool complete = i0 + kT <= n;
        const int64_t* src = p.idx + ((long long)b * n + i0) * m;
        // ---- warm the L2: this tile's position-table indices and mask (wanted after the de-duplication) and the
        //      index rows of this warp's next tile
        {
            const long long toff = ((long long)b * n + i0) * m;
            if (lane * 16 < E) {
                if (p.table) prefetch_l2(p.pe_idx + toff + lane * 16);
                if (p.mask) prefetch_l2(p.mask + toff + lane * 16);
            }
            const unsigned nt = task + nwarps;
            if (nt < total && lane * 16 < E) {
                const int nb = (int)(nt / (unsigned)p.tiles);
                const long long noff = ((long long)nb * n + (long long)(nt - (unsigned)nb * (unsigned)p.tiles) * kT) * m;
                prefetch_l2(p.idx + noff + lane * 16);
            }
        }
        // ---- the tile's indices
        __syncwarp();
        {
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
        bool rowdup = false;
        if (identical) {
            const int* ring32 = reinterpret_cast<const int*>(ring);
            for (int r = lane; r < m; r += 32) tok_s[r] = ring32[2 * r];
        } else {
            U = dedup_tile(ds, ring, lut, E, m, i0, n, true, &rowdup, lane);
        }
        __syncwarp();
        const int nchunks = U > 0 ? (U + kUC - 1) / kUC : 1;
        // position-table index (bits 0..30; all ones = none) and mask bit (bit 31 = masked out) of every edge of
        // this lane: the same for all heads, requested now so that they arrive while head 0 stages its rows
        const int valid = min(kT, n - i0) * m;
        unsigned pm[kEPL];
        {
            const int64_t* pe_t = p.table ? p.pe_idx + ((long long)b * n + i0) * m : nullptr;
            const int64_t* mask_t = p.mask ? p.mask + ((long long)b * n + i0) * m : nullptr;
#pragma unroll
            for (int k = 0; k < kEPL; ++k) {
                const int x = lane + 32 * k;
                unsigned v = 0x7fffffffu;
                if (x < valid) {
                    if (pe_t) {
                        const long long pi = pe_t[x];
                        if (pi >= 0 && pi < p.table_rows) v = (unsigned)pi;
                    }
                    if (mask_t && mask_t[x] == 0) v |= 0x80000000u;
                }
                pm[k] = v;
            }
        }
        // the tile's [8][m] rows of a dense bias are contiguous: they can travel as 16-byte pieces
        const bool bias_async = p.bias != nullptr && complete && ((m * (int)sizeof(T)) & 15) == 0 && p.bias_aligned;

        for (int g = 0; g < heads; ++g) {
            const long long bh = (long long)b * heads + g;
            const T* Kh = Kg + (long long)b * p.gs.x_batch + (long long)g * p.gs.x_head;
            const T* Vh = Vg + (long long)b * p.gs.x_batch + (long long)g * p.gs.x_head;
            const T* Qt = Qg + (long long)b * p.gs.y_batch + (long long)g * p.gs.y_head + (long long)i0 * p.gs.y_row;
            // 16-bit inputs: the query fragments of the score product come straight from global memory; requested
            // here, they arrive while the key rows are staged
            unsigned yb[2][2] = {{0u, 0u}, {0u, 0u}};
            if (!kIsFloat) {
                const int yg = lane >> 2, yt = lane & 3;
                if (i0 + yg < n) {
                    const unsigned* yrow = reinterpret_cast<const unsigned*>(Qt + (long long)yg * p.gs.y_row);
#pragma unroll
                    for (int ks = 0; ks < 2; ++ks) {
                        yb[ks][0] = yrow[8 * ks + yt];
                        yb[ks][1] = yrow[8 * ks + 4 + yt];
                    }
                }
            }
            // ================= scores =================
            float oreg[kEPL];
#pragma unroll
            for (int k = 0; k < kEPL; ++k) oreg[k] = 0.f;
            for (int ch = 0; ch < nchunks; ++ch) {
                const int u0 = ch * kUC;
                const int Uc = max(0, min(kUC, U - u0));
                __syncwarp();
                if (ch == 0 && bias_async) {
                    const T* bias_t = static_cast<const T*>(p.bias) + (bh * n + i0) * m;
                    T* Bt = reinterpret_cast<T*>(Wd);           // [8 m] in edge order; the weight tile is free until the output phase
                    for (int z = lane; z < E / kPer; z += 32) cp_async16_ca(Bt + z * kPer, bias_t + z * kPer);
                }
                stage(Kh, u0, Uc, identical, true);
                if (kIsFloat && ch == 0) {
                    // the tile's query rows -> Ys (fp32, row stride kYLD)
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const int z = lane + 32 * k;
                        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (i0 + (z >> 3) < n) v = ld4(Qt + (long long)(z >> 3) * p.gs.y_row + (z & 7) * 4);
                        *reinterpret_cast<float4*>(Ys + (z >> 3) * kYLD + (z & 7) * 4) = v;
                    }
                }
                cp_async_wait<0>();
                __syncwarp();
                float* Sdst = identical ? P : Sb;
                if (kIsFloat) {
                    dot_product_mma<true>(identical ? da_p : da, (Uc + 15) >> 4);
                } else {
                    dot_product16<T>(Xraw, yb, Sdst, (Uc + 15) >> 4, lane);
                }
                __syncwarp();
                // every edge whose neighbour is in this round picks its score (identical rows: already in place)
                if (!identical) {
#pragma unroll
                    for (int k = 0; k < kEPL; ++k) {
                        const int x = lane + 32 * k;
                        if (x < E) {
                            const int q = (int)((qpack >> (3 * k)) & 7ull);
                            const unsigned short sl = lut[x];
                            const int rel = (int)sl - u0;
                            if (sl != kSkip && rel >= 0 && rel < Uc) oreg[k] = Sb[q * kWLD + rel];
                        }
                    }
                }
            }
            // the row buffer is free again: the first round of VALUE rows travels while the logits are finished
            // and the softmax runs
            __syncwarp();
            stage(Vh, 0, max(0, min(kUC, U)), identical, false);
            // ================= logits: + bias, + mask; -> P[row][neighbour] =================
            {
                // the tile's rows of the bias are contiguous: element (row q, neighbour j) is x = q m + j
                const T* bias_t = (p.bias && !bias_async) ? static_cast<const T*>(p.bias) + (bh * n + i0) * m : nullptr;
                const T* Bt = reinterpret_cast<const T*>(Wd);
                const T* table_g = static_cast<const T*>(p.table) + g;
#pragma unroll
                for (int k = 0; k < kEPL; ++k) {
                    const int x = lane + 32 * k;
                    if (x < E) {
                        const int q = (int)((qpack >> (3 * k)) & 7ull);
                        const int j = x - q * m;
                        float lg = identical ? P[q * kWLD + j] : oreg[k];
                        if (x < valid) {
                            if (bias_async) lg += Elem<T>::up(Bt[x]);
                            else if (bias_t) lg += Elem<T>::up(bias_t[x]);
                            const unsigned pi = pm[k] & 0x7fffffffu;
                            if (p.table && pi != 0x7fffffffu) lg += Elem<T>::up(table_g[(long long)pi * heads]);
                            if (pm[k] & 0x80000000u) lg -= 100.f;
                        }
                        P[q * kWLD + j] = lg;
                    }
                }
            }
            // blank-token logit of row srow: <query, blank_k>, 8 channels per lane
            float blank = -INFINITY;
            if (p.blank_k) {
                float s = 0.f;
                if (i0 + srow < n) {
                    const T* qrow = Qt + (long long)srow * p.gs.y_row + part * 8;
                    const T* bk = static_cast<const T*>(p.blank_k) + g * kC + part * 8;
#pragma unroll
                    for (int c = 0; c < 8; ++c) s += Elem<T>::up(qrow[c]) * Elem<T>::up(bk[c]);
                }
                s += __shfl_xor_sync(kFull, s, 1);
                s += __shfl_xor_sync(kFull, s, 2);
                blank = s;
            }
            __syncwarp();
            // ================= softmax over the m neighbours (and the blank token) of row srow =================
            float pb = 0.f;                                   // probability of the blank token
            {
                float* prow = P + srow * kWLD;
                float mx = blank;
                for (int j = part; j < m; j += 4) mx = fmaxf(mx, prow[j]);
                mx = fmaxf(mx, __shfl_xor_sync(kFull, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(kFull, mx, 2));
                float sum = 0.f;
                for (int j = part; j < m; j += 4) {
                    const float e = __expf(prow[j] - mx);
                    prow[j] = e;
                    sum += e;
                }
                sum += __shfl_xor_sync(kFull, sum, 1);
                sum += __shfl_xor_sync(kFull, sum, 2);
                const float eb = p.blank_k ? __expf(blank - mx) : 0.f;
                const float inv = 1.f / (sum + eb);
                for (int j = part; j < m; j += 4) prow[j] *= inv;
                pb = eb * inv;
            }
            __syncwarp();
            // ================= output =================
            float acc[2][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[0][i] = acc[1][i] = 0.f;
            for (int ch = 0; ch < nchunks; ++ch) {
                const int u0 = ch * kUC;
                const int Uc = max(0, min(kUC, U - u0));
                const int rows8 = (Uc + 7) & ~7;
                __syncwarp();
                if (ch > 0) stage(Vh, u0, Uc, identical, false);
                // ---- dense probabilities of this round, by slot (identical rows in fp32: the probability tile
                //      itself is that matrix, slot = neighbour)
                const bool p_is_wd = kIsFloat && identical;
                if (p_is_wd) {
                    // columns m .. 47 of P are never written by the softmax: the product must not see stale values
                    for (int z = lane; z < kT * (kUC - m); z += 32) P[(z / (kUC - m)) * kWLD + m + z % (kUC - m)] = 0.f;
                } else if (kIsFloat) {
                    for (int z = lane; z < kT * kWLD / 4; z += 32)
                        reinterpret_cast<float4*>(Wd)[z] = make_float4(0.f, 0.f, 0.f, 0.f);
                } else {
                    for (int z = lane; z < kT * kWLD16 * 2 / 16; z += 32)
                        reinterpret_cast<float4*>(Wd16)[z] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
                __syncwarp();
                if (p_is_wd) {
                } else if (identical || !rowdup) {
#pragma unroll
                    for (int k = 0; k < kEPL; ++k) {
                        const int x = lane + 32 * k;
                        if (x < E) {
                            const int q = (int)((qpack >> (3 * k)) & 7ull);
                            const int j = x - q * m;
                            int rel = j;
                            bool in = ch == 0;
                            if (!identical) {
                                const unsigned short sl = lut[x];
                                rel = (int)sl - u0;
                                in = sl != kSkip && rel >= 0 && rel < Uc;
                            }
                            if (in) {
                                const float w = P[q * kWLD + j];
                                if (kIsFloat) Wd[q * kWLD + rel] = w;
                                else Wd16[q * kWLD16 + rel] = Elem<T>::down(w);
                            }
                        }
                    }
                } else if (lane < kT) {
                    // some row repeats a neighbour: one lane per row adds its probabilities in column order
                    float* tmp = Sb + lane * kWLD;              // the score tile is free: fp32 sums by slot
                    for (int r = 0; r < Uc; ++r) tmp[r] = 0.f;
#pragma unroll 1
                    for (int j = 0; j < m; ++j) {
                        const unsigned short sl = lut[lane * m + j];
                        const int rel = (int)sl - u0;
                        if (sl != kSkip && rel >= 0 && rel < Uc) tmp[rel] += P[lane * kWLD + j];
                    }
                    for (int r = 0; r < Uc; ++r) {
                        if (kIsFloat) Wd[lane * kWLD + r] = tmp[r];
                        else Wd16[lane * kWLD16 + r] = Elem<T>::down(tmp[r]);
                    }
                }
                cp_async_wait<0>();
                __syncwarp();
                if (kIsFloat) sum_product_mma<true>(p_is_wd ? sa_p : sa, rows8, acc);
                else sum_product16<T>(Xraw, Wd16, (Uc + 15) >> 4, lane, acc);
            }
            // D fragments -> output tile in the score tile -> + blank probability x blank value -> 16-byte stores
            {
                float* Ot = Sb;
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
#pragma unroll
                for (int a = 0; a < 2; ++a) {
                    const int q = 2 * qi + a;
                    // the blank probability of row q lives in the lanes 4 q .. 4 q + 3
                    const float pq = __shfl_sync(kFull, pb, 4 * q);
                    if (i0 + q < n) {
                        float4 v = *reinterpret_cast<const float4*>(Ot + q * kOLD + ci * 4);
                        if (p.blank_v) {
                            const float4 bv = ld4(static_cast<const T*>(p.blank_v) + g * kC + ci * 4);
                            v.x += pq * bv.x;  v.y += pq * bv.y;  v.z += pq * bv.z;  v.w += pq * bv.w;
                        }
                        st4(Og + (bh * n + i0 + q) * kC + ci * 4, v);
                    }
                }
                __syncwarp();
            }
        }
    }
}

template <typename T>
int fused_t(FusedParams p, cudaStream_t s) {
    p.tiles = (p.n + kT - 1) / kT;
    if ((long long)p.batch * p.tiles > 0x7fffffffLL) return CLUSTEN_ERR_SHAPE;
    const size_t smem = size_t(kWarps) * FusedSmem<T>::kTotal;
    auto kernel = p.m == kMmax ? fused_attention_kernel<T, true> : fused_attention_kernel<T, false>;
    const int per_sm = resident_ctas(reinterpret_cast<const void*>(kernel), 32 * kWarps, smem);
    if (per_sm < 0) return per_sm;
    long long grid = (long long)sm_count() * per_sm;
    const long long need = ((long long)p.batch * p.tiles + kWarps - 1) / kWarps;
    if (grid > need) grid = need;
    ScopedKernelTimer timer("fused_attention", s);
    kernel<<<(int)grid, 32 * kWarps, smem, s>>>(p);
    note_launch();
    return check_launch();
}

}  // namespace

bool fused_attention_supported(int dtype, int n, int m, int c) {
    if (dtype != CLUSTEN_F32 && dtype != CLUSTEN_F16 && dtype != CLUSTEN_BF16) return false;
    return c == kC && m >= 1 && m <= kMmax && n >= 1 && n <= 65000;
}

int launch_fused_attention(int dtype, const void* q, const void* k, const void* v, const int64_t* idx, const void* bias,
                           const void* table, const int64_t* pe_idx, int table_rows, const int64_t* mask,
                           const void* blank_k, const void* blank_v, void* out, int b, int h, int n, int m,
                           GatherStrides gs, cudaStream_t s) {
    if (gs.x_row == 0) {
        gs.x_batch = (long long)h * n * kC;  gs.x_head = (long long)n * kC;  gs.x_row = kC;
    }
    if (gs.y_row == 0) {
        gs.y_batch = (long long)h * n * kC;  gs.y_head = (long long)n * kC;  gs.y_row = kC;
    }
    FusedParams p{};
    p.q = q;  p.k = k;  p.v = v;  p.idx = idx;  p.bias = bias;  p.table = table;  p.pe_idx = pe_idx;
    p.table_rows = table_rows;  p.mask = mask;  p.blank_k = blank_k;  p.blank_v = blank_v;  p.out = out;
    p.batch = b;  p.heads = h;  p.n = n;  p.m = m;  p.gs = gs;
    p.bias_aligned = bias != nullptr && reinterpret_cast<uintptr_t>(bias) % 16 == 0 &&
                     ((long long)n * m * dtype_size(dtype)) % 16 == 0;
    switch (dtype) {
        case CLUSTEN_F32: return fused_t<float>(p, s);
        case CLUSTEN_F16: return fused_t<__half>(p, s);
        case CLUSTEN_BF16: return fused_t<__nv_bfloat16>(p, s);
        default: return CLUSTEN_ERR_DTYPE;
    }
}

}  // namespace clusten
