// Backward of the weighted gather-add.
//
//   dw[n, i]            = <dy[n, :], tables[idx[n, i], :]>      (reference: indexed_inner_product,
//                          gather/cuda/extension/gather_kernel_fp32.cu:94-157)
//   dtables[idx[n, i]] += w[n, i] * dy[n, :]                     (reference: weighted_vector_scatter_add,
//                          gather_kernel_fp32.cu:49-92, one scalar atomicAdd per element)
//
// dw: one warp per token, dy[n] held in registers in the same 16-byte-vector layout as the rows;
// each lane keeps its partial dot product of 32 consecutive rows in 32 registers, then one
// 31-shuffle transpose-reduce hands lane j the full sum of row j: one coalesced 128-byte store
// per 32 rows instead of a 5-shuffle reduction and a shared-memory atomic per row.
//
// dtables, any index list: one warp per token, dy[n] in registers, one 16-byte vector reduction
// (red.global.add.v4.f32) per lane per row -- a quarter of the reference's atomic count, resolved
// in L2.
//
// dtables, layer-structured index list (I = T*m, entry (n, t*m+c) lands in table t): entries are
// counting-sorted per table into scratch by a stable in-CTA sort, then the segmented form of the
// forward gather kernel sums each output row's terms in ascending (n, c) order from dy and
// writes the row once: no atomics on the output, no memset, bit-reproducible, and equal to the
// CPU oracle's fmaf chain.
#include <mutex>

#include "common.cuh"

namespace lffn {

int launch_gather_segmented(const int32_t *idx, const float *w, const float *src, float *out, int64_t n_out,
                            const int2 *seg, int64_t n_src, int d, cudaStream_t st);  // gather_fwd.cu

// ---- dw ----------------------------------------------------------------------------------------
#ifndef LFFN_BWW_THREADS
#define LFFN_BWW_THREADS 128
#endif
#ifndef LFFN_BWW_MINBLOCKS
#define LFFN_BWW_MINBLOCKS 3
#endif
#ifndef LFFN_BWW_U_NARROW
#define LFFN_BWW_U_NARROW 4
#endif
#ifndef LFFN_BWW_U_WIDE
#define LFFN_BWW_U_WIDE 2
#endif

template <typename TableT, int VPL, int U, bool FULLV>
__global__ void __launch_bounds__(LFFN_BWW_THREADS, LFFN_BWW_MINBLOCKS)
    gather_bwd_weights_kernel(const int32_t *__restrict__ idx, const float *__restrict__ dy,
                              const TableT *__restrict__ tables, float *__restrict__ dw, long long N, int I,
                              long long S, int d, int col0, int accumulate, int i0, int icnt, uint32_t *status) {
    // i0/icnt: the slice of each token's index list this launch covers (see launch_bww_vpl)
    constexpr int EPV = Elem<TableT>::PER_VEC;
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    const long long warp0 = (long long)blockIdx.x * wpb + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * wpb;
    const int row_vecs = d / EPV;
    const int nvec = min(row_vecs - col0, VPL * 32);
    const uint4 *tv = reinterpret_cast<const uint4 *>(tables) + col0;
    bool bad = false;

    for (long long n = warp0; n < N; n += nwarps) {
        float g[VPL][EPV];
        const float *dyr = dy + n * d + (long long)col0 * EPV;
#pragma unroll
        for (int v = 0; v < VPL; v++) {
            const int c = lane + 32 * v;
#pragma unroll
            for (int q = 0; q < EPV / 4; q++) {
                float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
                if (c < nvec) t = __ldg(reinterpret_cast<const float4 *>(dyr + c * EPV + 4 * q));
                g[v][4 * q] = t.x;
                g[v][4 * q + 1] = t.y;
                g[v][4 * q + 2] = t.z;
                g[v][4 * q + 3] = t.w;
            }
        }
        const int32_t *ip = idx + n * I + i0;
        int next_i = lane < icnt ? __ldg(ip + lane) : 0;
        for (int g0 = 0; g0 < icnt; g0 += 32) {
            const int cnt = min(32, icnt - g0);
            const int my_i = next_i;
            if (g0 + 32 + lane < icnt) next_i = __ldg(ip + g0 + 32 + lane);
            // branch-free: rows past the list end or out of range read a substitute row (row 0) and their sums are
            // discarded; every lane checks the one index it loaded, the loop broadcasts checked indices only
            const bool mine_in_range = (unsigned long long)(long long)my_i < (unsigned long long)S;
            bad |= (lane < cnt) && !mine_in_range;
            const int san_i = mine_in_range ? my_i : 0;
            float p[32];
#pragma unroll
            for (int j0 = 0; j0 < 32; j0 += U) {
                uint4 buf[U][VPL];
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int j = j0 + u;
                    const int r = __shfl_sync(FULL, san_i, j);
                    const uint4 *row = tv + (long long)r * row_vecs;
#pragma unroll
                    for (int v = 0; v < VPL; v++) {
                        const int c = lane + 32 * v;
                        buf[u][v] = FULLV ? ld_row16(row + c) : ld_row16_pred(row + c, c < nvec);
                    }
                }
#pragma unroll
                for (int u = 0; u < U; u++) {
                    float s = 0.f;
#pragma unroll
                    for (int v = 0; v < VPL; v++) {
                        float f[EPV];
                        Elem<TableT>::unpack(buf[u][v], f);
#pragma unroll
                        for (int e = 0; e < EPV; e++) s = fmaf(g[v][e], f[e], s);
                    }
                    p[j0 + u] = s;
                }
            }
            // transpose-reduce: after the 5 rounds lane j holds sum over lanes of p[j]
#pragma unroll
            for (int s = 16; s >= 1; s >>= 1) {
                const bool up = (lane & s) != 0;
#pragma unroll
                for (int j = 0; j < s; j++) {
                    const float send = up ? p[j] : p[j + s];
                    const float keep = up ? p[j + s] : p[j];
                    p[j] = keep + __shfl_xor_sync(FULL, send, s);
                }
            }
            if (lane < cnt) {
                const bool in_range = (unsigned long long)(long long)my_i < (unsigned long long)S;
                const float val = in_range ? p[0] : 0.f;
                float *o = dw + n * I + i0 + g0 + lane;
                *o = accumulate ? (*o + val) : val;
            }
        }
    }
    if (bad) atomicOr(status, LFFN_STATUS_INDEX_RANGE);
}

template <typename TableT, int VPL>
static int launch_bww_vpl(const int32_t *idx, const float *dy, const void *tables, float *dw, int64_t N, int I,
                          int64_t S, int d, int col0, cudaStream_t st) {
    constexpr int U = (VPL <= 3) ? LFFN_BWW_U_NARROW : LFFN_BWW_U_WIDE;
    constexpr int THREADS = LFFN_BWW_THREADS;
    const int nvec_here = min(d / Elem<TableT>::PER_VEC - col0, VPL * 32);
    auto kern = nvec_here == VPL * 32 ? gather_bwd_weights_kernel<TableT, VPL, U, true>
                                      : gather_bwd_weights_kernel<TableT, VPL, U, false>;
    int per_sm = 0;
    LFFN_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, THREADS, 0));
    if (per_sm < 1) per_sm = 1;
    const long long want = (N + THREADS / 32 - 1) / (THREADS / 32);
    long long grid = (long long)num_sms() * per_sm;
    if (grid > want) grid = want;
    if (grid < 1) grid = 1;
    // Long lists over table sets beyond L2 are consumed in slices, one launch per slice over all tokens, which
    // keeps the warps aligned along the list and each launch's rows L2-resident (same reason as in the forward
    // gather); every dw element belongs to exactly one slice, so nothing else changes.
    int slices = 1;
    if (I >= 512) {
        const double table_bytes = (double)S * d * sizeof(TableT);
        if (table_bytes > 256e6) slices = (int)(table_bytes / LFFN_GATHER_SLICE_BYTES);
        if (slices > I / 128) slices = I / 128;
        if (slices < 1) slices = 1;
    }
    const int per = slices == 1 ? I : ((I + slices - 1) / slices + 31) / 32 * 32;
    uint32_t *status = status_word();
    LFFN_REQUIRE(status != nullptr, LFFN_ERR_CUDA, "cannot locate the device status word");
    for (int i0 = 0; i0 < I; i0 += per) {
        const int icnt = I - i0 < per ? I - i0 : per;
        kern<<<(unsigned)grid, THREADS, 0, st>>>(idx, dy, static_cast<const TableT *>(tables), dw, N, I, S, d, col0,
                                                 col0 > 0 ? 1 : 0, i0, icnt, status);
        LFFN_CHECK_CUDA(cudaGetLastError());
    }
    return LFFN_OK;
}

template <typename TableT>
static int launch_bww_typed(const int32_t *idx, const float *dy, const void *tables, float *dw, int64_t N, int I,
                            int64_t S, int d, cudaStream_t st) {
    constexpr int EPV = Elem<TableT>::PER_VEC;
    const int row_vecs = d / EPV;
    constexpr int MAXV = 6;
    for (int col0 = 0; col0 < row_vecs; col0 += MAXV * 32) {
        const int nvec = min(row_vecs - col0, MAXV * 32);
        const int vpl = (nvec + 31) / 32;
        int rc;
        switch (vpl) {
            case 1: rc = launch_bww_vpl<TableT, 1>(idx, dy, tables, dw, N, I, S, d, col0, st); break;
            case 2: rc = launch_bww_vpl<TableT, 2>(idx, dy, tables, dw, N, I, S, d, col0, st); break;
            case 3: rc = launch_bww_vpl<TableT, 3>(idx, dy, tables, dw, N, I, S, d, col0, st); break;
            case 4: rc = launch_bww_vpl<TableT, 4>(idx, dy, tables, dw, N, I, S, d, col0, st); break;
            default: rc = launch_bww_vpl<TableT, 6>(idx, dy, tables, dw, N, I, S, d, col0, st); break;
        }
        if (rc != LFFN_OK) return rc;
    }
    return LFFN_OK;
}

int launch_gather_bwd_weights(const int32_t *idx, const float *dy, const void *tables, int table_dtype, float *dw,
                              int64_t N, int I, int64_t S, int d, cudaStream_t st) {
    if (table_dtype == LFFN_F32) return launch_bww_typed<float>(idx, dy, tables, dw, N, I, S, d, st);
    if (table_dtype == LFFN_BF16) return launch_bww_typed<__nv_bfloat16>(idx, dy, tables, dw, N, I, S, d, st);
    set_error("gather_bwd_weights: unknown table dtype %d", table_dtype);
    return LFFN_ERR_INVALID_ARG;
}

// ---- dtables, any index list: vector reductions in L2 ---------------------------------------------
__device__ __forceinline__ void red_add_v4(float *p, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <int VPL>
__global__ void __launch_bounds__(256) gather_bwd_tables_red_kernel(const int32_t *__restrict__ idx,
                                                                    const float *__restrict__ w,
                                                                    const float *__restrict__ dy,
                                                                    float *__restrict__ dtables, long long N, int I,
                                                                    long long S, int d, int col0, uint32_t *status) {
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    const long long warp0 = (long long)blockIdx.x * wpb + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * wpb;
    const int row_vecs = d / 4;
    const int nvec = min(row_vecs - col0, VPL * 32);
    bool bad = false;
    for (long long n = warp0; n < N; n += nwarps) {
        float4 g[VPL];
        const float *dyr = dy + n * d + (long long)col0 * 4;
#pragma unroll
        for (int v = 0; v < VPL; v++) {
            const int c = lane + 32 * v;
            g[v] = c < nvec ? __ldg(reinterpret_cast<const float4 *>(dyr) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        for (int g0 = 0; g0 < I; g0 += 32) {
            const int cnt = min(32, I - g0);
            const int my_i = lane < cnt ? __ldg(idx + n * I + g0 + lane) : 0;
            const float my_w = lane < cnt ? __ldg(w + n * I + g0 + lane) : 0.f;
            for (int j = 0; j < cnt; j++) {
                const int r = __shfl_sync(FULL, my_i, j);
                const float ww = __shfl_sync(FULL, my_w, j);
                if ((unsigned long long)(long long)r >= (unsigned long long)S) {
                    bad = true;
                    continue;
                }
                float *row = dtables + (long long)r * d + (long long)col0 * 4;
#pragma unroll
                for (int v = 0; v < VPL; v++) {
                    const int c = lane + 32 * v;
                    if (c < nvec) red_add_v4(row + c * 4, ww * g[v].x, ww * g[v].y, ww * g[v].z, ww * g[v].w);
                }
            }
        }
    }
    if (bad) atomicOr(status, LFFN_STATUS_INDEX_RANGE);
}

template <int VPL>
static int launch_red_vpl(const int32_t *idx, const float *w, const float *dy, float *dtables, int64_t N, int I,
                          int64_t S, int d, int col0, cudaStream_t st) {
    constexpr int THREADS = 256;
    auto kern = gather_bwd_tables_red_kernel<VPL>;
    int per_sm = 0;
    LFFN_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, THREADS, 0));
    if (per_sm < 1) per_sm = 1;
    const long long want = (N + THREADS / 32 - 1) / (THREADS / 32);
    long long grid = (long long)num_sms() * per_sm;
    if (grid > want) grid = want;
    if (grid < 1) grid = 1;
    uint32_t *status = status_word();
    LFFN_REQUIRE(status != nullptr, LFFN_ERR_CUDA, "cannot locate the device status word");
    kern<<<(unsigned)grid, THREADS, 0, st>>>(idx, w, dy, dtables, N, I, S, d, col0, status);
    LFFN_CHECK_CUDA(cudaGetLastError());
    return LFFN_OK;
}

int launch_gather_bwd_tables(const int32_t *idx, const float *w, const float *dy, float *dtables, int64_t N, int I,
                             int64_t S, int d, cudaStream_t st) {
    LFFN_CHECK_CUDA(cudaMemsetAsync(dtables, 0, (size_t)S * d * sizeof(float), st));
    const int row_vecs = d / 4;
    constexpr int MAXV = 8;
    for (int col0 = 0; col0 < row_vecs; col0 += MAXV * 32) {
        const int nvec = min(row_vecs - col0, MAXV * 32);
        const int vpl = (nvec + 31) / 32;
        int rc;
        if (vpl <= 1) rc = launch_red_vpl<1>(idx, w, dy, dtables, N, I, S, d, col0, st);
        else if (vpl <= 2) rc = launch_red_vpl<2>(idx, w, dy, dtables, N, I, S, d, col0, st);
        else if (vpl <= 4) rc = launch_red_vpl<4>(idx, w, dy, dtables, N, I, S, d, col0, st);
        else if (vpl <= 6) rc = launch_red_vpl<6>(idx, w, dy, dtables, N, I, S, d, col0, st);
        else rc = launch_red_vpl<8>(idx, w, dy, dtables, N, I, S, d, col0, st);
        if (rc != LFFN_OK) return rc;
    }
    return LFFN_OK;
}

// ---- dtables, layer-structured index list: stable per-table counting sort + segmented reduction ----
constexpr int SORT_THREADS = 512;
constexpr int SORT_MAX_ROWS = 16384;
constexpr long long SORT_WARP_RANGE_ENTRIES = 65536;  // ... and only for tables with at most this many entries
constexpr int SORT_WARP_RANGE_ROWS = 2048;  // up to here every warp keeps its own counters: 16 x rows x 4 B of shared memory

// scratch layout: seg int2[T*rows] | ent_n int32[T*Ne] | ent_w float[T*Ne],  Ne = N*m
struct SortedScratch {
    int2 *seg;
    int32_t *ent_n;
    float *ent_w;
};
static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }
size_t sorted_scratch_bytes(int64_t N, int T, int m, int rows) {
    const size_t ne = (size_t)N * m * T;
    return align256((size_t)T * rows * sizeof(int2)) + align256(ne * 4) + align256(ne * 4);
}
static SortedScratch carve(void *scratch, int64_t N, int T, int m, int rows) {
    char *p = static_cast<char *>(scratch);
    const size_t ne = (size_t)N * m * T;
    SortedScratch s;
    s.seg = reinterpret_cast<int2 *>(p);
    p += align256((size_t)T * rows * sizeof(int2));
    s.ent_n = reinterpret_cast<int32_t *>(p);
    p += align256(ne * 4);
    s.ent_w = reinterpret_cast<float *>(p);
    return s;
}

// One CTA sorts the N*m entries of one table by row, keeping ascending (n, c) order inside a row.
//
// WARP_RANGES (rows <= SORT_WARP_RANGE_ROWS): every warp owns one contiguous range of the table's entries.  The
// counting pass fills counts[warp][row]; an exclusive scan over (row, warp) turns them into the first output slot of
// each warp's entries of each row; the placement pass then runs without any CTA-wide barrier, every warp walking its
// range in order with its own cursors.  Stability: a warp's entries all come after those of the warps before it,
// and inside a warp the 32 entries of a step are ranked by lane.
// Otherwise (many rows: the per-warp counters would not fit in shared memory) one shared cursor per row and the
// warps take turns, in entry order, 512 entries per step.
template <bool WARP_RANGES>
__global__ void __launch_bounds__(SORT_THREADS) sort_table_entries_kernel(const int32_t *__restrict__ idx,
                                                                          const float *__restrict__ w, long long N,
                                                                          int T, int m, int rows, int2 *seg,
                                                                          int32_t *ent_n, float *ent_w,
                                                                          uint32_t *status) {
    extern __shared__ int cursor[];  // WARP_RANGES: [NW][rows] counts, then write offsets; else [rows]
    __shared__ int warp_sums[SORT_THREADS / 32];
    constexpr int NW = SORT_THREADS / 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long Ne = N * m;
    const int I = T * m;
    bool bad = false;
    // entries [e_lo, e_hi) of every table belong to this warp (WARP_RANGES); multiples of 32 except at the end
    const long long per_warp = ((Ne + NW - 1) / NW + 31) / 32 * 32;
    const long long e_lo = min(Ne, per_warp * warp), e_hi = min(Ne, e_lo + per_warp);
    const int ncnt = WARP_RANGES ? NW * rows : rows;
    for (int t = blockIdx.x; t < T; t += gridDim.x) {
        for (int i = tid; i < ncnt; i += SORT_THREADS) cursor[i] = 0;
        __syncthreads();
        const int32_t *col = idx + (long long)t * m;
        if constexpr (WARP_RANGES) {
            int *mine = cursor + warp * rows;
            for (long long e = e_lo + lane; e < e_hi; e += 32) {
                const long long n = e / m;
                const int c = (int)(e - n * m);
                const int key = __ldg(col + n * I + c) - t * rows;
                if ((unsigned)key < (unsigned)rows) atomicAdd(&mine[key], 1);
                else bad = true;
            }
        } else {
            for (long long e = tid; e < Ne; e += SORT_THREADS) {
                const long long n = e / m;
                const int c = (int)(e - n * m);
                const int key = __ldg(col + n * I + c) - t * rows;
                if ((unsigned)key < (unsigned)rows) atomicAdd(&cursor[key], 1);
                else bad = true;
            }
        }
        __syncthreads();
        // exclusive scan over the rows: each thread owns a contiguous chunk of rows (all warps' counts of a row
        // are consecutive in the order of the scan)
        const int chunk = (rows + SORT_THREADS - 1) / SORT_THREADS;
        const int b = min(tid * chunk, rows), e2 = min(b + chunk, rows);
        int local = 0;
        for (int i = b; i < e2; i++) {
            if constexpr (WARP_RANGES) {
                for (int ws = 0; ws < NW; ws++) local += cursor[ws * rows + i];
            } else {
                local += cursor[i];
            }
        }
        int incl = local;
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) {
            const int v = __shfl_up_sync(FULL, incl, s);
            if (lane >= s) incl += v;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int v = lane < NW ? warp_sums[lane] : 0;
#pragma unroll
            for (int s = 1; s < 32; s <<= 1) {
                const int u = __shfl_up_sync(FULL, v, s);
                if (lane >= s) v += u;
            }
            if (lane < NW) warp_sums[lane] = v;  // inclusive sums of warps
        }
        __syncthreads();
        int run = incl - local + (warp > 0 ? warp_sums[warp - 1] : 0);
        const long long tbase = (long long)t * Ne;
        for (int i = b; i < e2; i++) {
            if constexpr (WARP_RANGES) {
                const int first = run;
                for (int ws = 0; ws < NW; ws++) {
                    const int cnt = cursor[ws * rows + i];
                    cursor[ws * rows + i] = run;
                    run += cnt;
                }
                seg[(long long)t * rows + i] = make_int2((int)(tbase + first), run - first);
            } else {
                const int cnt = cursor[i];
                seg[(long long)t * rows + i] = make_int2((int)(tbase + run), cnt);
                cursor[i] = run;
                run += cnt;
            }
        }
        __syncthreads();
        if constexpr (WARP_RANGES) {
            int *mine = cursor + warp * rows;
            for (long long base = e_lo; base < e_hi; base += 32) {
                const long long e = base + lane;
                long long n = 0;
                int key = -1 - lane;  // unique per lane: matches nobody
                float ww = 0.f;
                if (e < e_hi) {
                    n = e / m;
                    const int c = (int)(e - n * m);
                    const int kk = __ldg(col + n * I + c) - t * rows;
                    if ((unsigned)kk < (unsigned)rows) {
                        key = kk;
                        ww = __ldg(w + n * I + (long long)t * m + c);
                    }
                }
                const unsigned peers = __match_any_sync(FULL, key);
                const int rank = __popc(peers & ((1u << lane) - 1u));
                const int leader = __ffs(peers) - 1;
                int basepos = 0;
                if (key >= 0 && rank == 0) {
                    basepos = mine[key];
                    mine[key] = basepos + __popc(peers);
                }
                __syncwarp();
                basepos = __shfl_sync(FULL, basepos, leader);
                if (key >= 0) {
                    const long long pos = tbase + basepos + rank;
                    ent_n[pos] = (int32_t)n;
                    ent_w[pos] = ww;
                }
            }
        } else {
            // stable placement, SORT_THREADS entries per step in entry order
            for (long long base = 0; base < Ne; base += SORT_THREADS) {
                const long long e = base + tid;
                long long n = 0;
                int key = -1 - lane;  // unique per lane: matches nobody
                float ww = 0.f;
                if (e < Ne) {
                    n = e / m;
                    const int c = (int)(e - n * m);
                    const int kk = __ldg(col + n * I + c) - t * rows;
                    if ((unsigned)kk < (unsigned)rows) {
                        key = kk;
                        ww = __ldg(w + n * I + (long long)t * m + c);
                    }
                }
                const unsigned peers = __match_any_sync(FULL, key);
                const int rank = __popc(peers & ((1u << lane) - 1u));
                const int leader = __ffs(peers) - 1;
                int basepos = 0;
                for (int ws = 0; ws < NW; ws++) {  // warps take their turn in entry order
                    if (warp == ws && key >= 0 && rank == 0) {
                        basepos = cursor[key];
                        cursor[key] = basepos + __popc(peers);
                    }
                    __syncthreads();
                }
                basepos = __shfl_sync(FULL, basepos, leader);
                if (key >= 0) {
                    const long long pos = tbase + basepos + rank;
                    ent_n[pos] = (int32_t)n;
                    ent_w[pos] = ww;
                }
            }
        }
        __syncthreads();
    }
    if (bad) atomicOr(status, LFFN_STATUS_STRUCTURE);
}

int launch_gather_bwd_tables_sorted(const int32_t *idx, const float *w, const float *dy, float *dtables, int64_t N,
                                    int T, int m, int rows, int d, void *scratch, size_t scratch_bytes,
                                    cudaStream_t st) {
    if (rows > SORT_MAX_ROWS) {
        set_error("gather_bwd_tables_sorted: %d rows per table exceeds %d; use lffn_gather_bwd_tables", rows,
                  SORT_MAX_ROWS);
        return LFFN_ERR_UNSUPPORTED;
    }
    if ((long long)N * m * T >= (1ll << 31)) {
        set_error("gather_bwd_tables_sorted: N*T*m = %lld entries exceed 2^31", (long long)N * m * T);
        return LFFN_ERR_UNSUPPORTED;
    }
    if (scratch == nullptr || scratch_bytes < sorted_scratch_bytes(N, T, m, rows)) {
        set_error("gather_bwd_tables_sorted: scratch of %zu bytes needed, %zu given", sorted_scratch_bytes(N, T, m, rows),
                  scratch_bytes);
        return LFFN_ERR_SCRATCH;
    }
    SortedScratch s = carve(scratch, N, T, m, rows);
#ifdef LFFN_SORT_NO_WARP_RANGES
    const bool warp_ranges = false;  // tuning builds: the shared-cursor placement for every shape
#else
    // per-warp ranges multiply the number of output streams by 16: worth it while a table's entries stay L2-resident
    // (measured: 32,768 entries per table 0.99 vs 1.07 ms; 147,456 entries per table 22.8 vs 20.8 ms)
    const bool warp_ranges = rows <= SORT_WARP_RANGE_ROWS && (long long)N * m <= SORT_WARP_RANGE_ENTRIES;
#endif
    const size_t smem = (size_t)rows * sizeof(int) * (warp_ranges ? SORT_THREADS / 32 : 1);
    auto kern = warp_ranges ? sort_table_entries_kernel<true> : sort_table_entries_kernel<false>;
    if (smem > 48 * 1024) LFFN_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int grid = T < 4 * num_sms() ? T : 4 * num_sms();
    uint32_t *status = status_word();
    LFFN_REQUIRE(status != nullptr, LFFN_ERR_CUDA, "cannot locate the device status word");
    kern<<<grid, SORT_THREADS, smem, st>>>(idx, w, N, T, m, rows, s.seg, s.ent_n, s.ent_w, status);
    LFFN_CHECK_CUDA(cudaGetLastError());
    return launch_gather_segmented(s.ent_n, s.ent_w, dy, dtables, (int64_t)T * rows, s.seg, N, d, st);
}

// ---- the same sorted table gradient for callers that cannot allocate device memory -------------------
// Its scratch is this fixed array instead of a caller buffer.  The array is part of the library image:
// every GPU that loads liblookupffn.so keeps these bytes reserved until the process exits.
constexpr size_t STATIC_SCRATCH_BYTES = LFFN_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

// Host code cannot use `g_static_scratch` as a pointer: in host code that name is only a handle for the
// runtime.  The real device address is asked for once per device (with that device current) and cached.
static int static_scratch_address(void **out) {
    static std::mutex mu;
    static void *addr[64] = {nullptr};
    int dev = 0;
    LFFN_CHECK_CUDA(cudaGetDevice(&dev));
    LFFN_REQUIRE(dev >= 0 && dev < 64, LFFN_ERR_UNSUPPORTED, "device ordinal %d", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (addr[dev] == nullptr) {
        void *p = nullptr;
        LFFN_CHECK_CUDA(cudaGetSymbolAddress((void **)&p, g_static_scratch));
        LFFN_REQUIRE(p != nullptr, LFFN_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        addr[dev] = p;
    }
    *out = addr[dev];
    return LFFN_OK;
}

}  // namespace lffn

extern "C" int lffn_gather_bwd_tables_sorted_static(const int32_t *idx, const float *w, const float *dy,
                                                    float *dtables, int64_t N, int32_t T, int32_t m, int32_t rows,
                                                    int32_t d, lffn_stream_t stream) {
    using namespace lffn;
    LFFN_REQUIRE(N >= 0 && T >= 1 && m >= 1 && rows >= 1 && d >= 1, LFFN_ERR_INVALID_ARG,
                 "gather_bwd_tables_sorted_static: bad sizes N=%lld T=%d m=%d rows=%d d=%d", (long long)N, T, m, rows, d);
    LFFN_REQUIRE(d % 4 == 0, LFFN_ERR_UNSUPPORTED, "gather_bwd_tables_sorted_static: d = %d must be a multiple of 4", d);
    LFFN_REQUIRE(dtables != nullptr && (N == 0 || (idx != nullptr && w != nullptr && dy != nullptr)),
                 LFFN_ERR_INVALID_ARG, "gather_bwd_tables_sorted_static: NULL buffer");
    LFFN_REQUIRE((reinterpret_cast<uintptr_t>(dtables) & 15u) == 0 && (reinterpret_cast<uintptr_t>(dy) & 15u) == 0,
                 LFFN_ERR_INVALID_ARG, "gather_bwd_tables_sorted_static: dtables and dy must be 16-byte aligned");
    LFFN_REQUIRE((long long)T * rows < (1ll << 31), LFFN_ERR_UNSUPPORTED,
                 "gather_bwd_tables_sorted_static: T*rows does not fit int32 indices");
    const size_t need = sorted_scratch_bytes(N, T, m, rows);
    LFFN_REQUIRE(need <= STATIC_SCRATCH_BYTES, LFFN_ERR_SCRATCH,
                 "gather_bwd_tables_sorted_static: this problem needs %zu bytes of scratch, the built-in array holds "
                 "%zu (N*T*m = %lld entries); use lffn_gather_bwd_tables_sorted with a caller buffer",
                 need, STATIC_SCRATCH_BYTES, (long long)N * T * m);
    void *scratch = nullptr;
    const int rc = static_scratch_address(&scratch);
    if (rc != LFFN_OK) return rc;
    return launch_gather_bwd_tables_sorted(idx, w, dy, dtables, N, T, m, rows, d, scratch, STATIC_SCRATCH_BYTES,
                                           static_cast<cudaStream_t>(stream));
}
