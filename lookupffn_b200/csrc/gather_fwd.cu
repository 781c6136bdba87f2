// Weighted gather-add, forward:  out[n, :] = sum_i w[n, i] * tables[idx[n, i], :] (+ bias).
//
// Replaces the reference's weighted_vector_gather_add kernels
// (gather/cuda/extension/gather_kernel_fp32.cu:3-47, gather_kernel_fp16.cu:6-62).
//
// Mapping: one warp owns one token.  A table row is d*eb bytes = nvec 16-byte vectors;
// lane l loads vectors l, l+32, ... (coalesced 512-byte warp requests) and keeps their fp32
// partial sums in registers for the whole index list, so every table byte is read once per
// use and the output row is written once.  Rows are processed U at a time so that U*VPL
// independent 16-byte loads per lane are in flight.  Indices and weights are read 32 at a
// time (one coalesced load per lane) and broadcast with shuffles; the next group of 32 is
// prefetched while the current one is consumed.  Every column's sum is one fmaf chain in
// index order, which is what the CPU oracle does, so fp32 results are bit-identical.
//
// The grid is a multiple of the SM count and warps walk tokens with a grid stride.  All
// resident warps sweep i = 0..I-1 at about the same pace, so at any time the rows being read
// come from a narrow band of tables, which keeps them L2-resident across the concurrently
// processed tokens even when the whole table set exceeds L2.
#include "common.cuh"

// Tuning constants (overridable at compile time): rows in flight per warp for narrow / medium /
// wide rows, threads per CTA and the minimum CTAs per SM the register allocation must allow.
#ifndef LFFN_GATHER_U_NARROW
#define LFFN_GATHER_U_NARROW 4
#endif
#ifndef LFFN_GATHER_U_MEDIUM
#define LFFN_GATHER_U_MEDIUM 2
#endif
#ifndef LFFN_GATHER_U_WIDE
#define LFFN_GATHER_U_WIDE 2
#endif
#ifndef LFFN_GATHER_THREADS
#define LFFN_GATHER_THREADS 128
#endif
#ifndef LFFN_GATHER_MINBLOCKS
#define LFFN_GATHER_MINBLOCKS 4
#endif

namespace lffn {

template <typename TableT, typename OutT, int VPL, int U, bool FULLV>
__global__ void __launch_bounds__(LFFN_GATHER_THREADS, LFFN_GATHER_MINBLOCKS) gather_fwd_kernel(const int32_t *__restrict__ idx, const float *__restrict__ w,
                                                         const TableT *__restrict__ tables, OutT *__restrict__ out,
                                                         long long N, int I, long long S, int d, int col0,
                                                         const float *__restrict__ bias, const int2 *__restrict__ seg,
                                                         uint32_t *status) {
    constexpr int EPV = Elem<TableT>::PER_VEC;
    const int lane = threadIdx.x & 31;
    const int warps_per_block = blockDim.x >> 5;
    const long long warp0 = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * warps_per_block;
    const int row_vecs = d / EPV;              // 16-byte vectors per table row
    const int nvec = min(row_vecs - col0, VPL * 32);  // vectors this launch covers, starting at col0
    const uint4 *tv = reinterpret_cast<const uint4 *>(tables) + col0;
    bool bad = false;

    for (long long n = warp0; n < N; n += nwarps) {
        float acc[VPL][EPV];
#pragma unroll
        for (int v = 0; v < VPL; v++)
#pragma unroll
            for (int e = 0; e < EPV; e++) acc[v][e] = 0.f;

        // dense [N, I] lists, or (segmented use: the sorted table-gradient reduction) list n = seg[n].x .. +seg[n].y
        const int32_t *ip = idx + n * I;
        const float *wp = w + n * I;
        if (seg != nullptr) {
            const int2 sg = __ldg(seg + n);
            ip = idx + sg.x;
            wp = w + sg.x;
            I = sg.y;
        }
        int my_i = 0;
        float my_w = 0.f;
        if (lane < I) {
            my_i = __ldg(ip + lane);
            my_w = __ldg(wp + lane);
        }
        for (int g0 = 0; g0 < I; g0 += 32) {
            const int cur_i = my_i;
            const float cur_w = my_w;
            if (g0 + 32 + lane < I) {  // prefetch the next 32 (idx, w) pairs
                my_i = __ldg(ip + g0 + 32 + lane);
                my_w = __ldg(wp + g0 + 32 + lane);
            }
            const int cnt = min(32, I - g0);
            // The loop body is branch-free: an entry past the end of the list, or with an index outside
            // [0, S), is replaced by (the group's first row, weight 0).  That row is part of the sum anyway,
            // so the substitute adds exactly nothing even when the row holds Inf or NaN.
            int safe = __shfl_sync(FULL, cur_i, 0);
            safe = (unsigned long long)(long long)safe < (unsigned long long)S ? safe : 0;
#pragma unroll 1
            for (int j0 = 0; j0 < cnt; j0 += U) {
                uint4 buf[U][VPL];
                float ww[U];
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int j = j0 + u;
                    int r = __shfl_sync(FULL, cur_i, j & 31);
                    float wj = __shfl_sync(FULL, cur_w, j & 31);
                    const bool in_list = j < cnt;
                    const bool in_range = (unsigned long long)(long long)r < (unsigned long long)S;
                    bad |= in_list && !in_range;
                    const bool ok = in_list && in_range;
                    r = ok ? r : safe;
                    ww[u] = ok ? wj : 0.f;
                    const uint4 *row = tv + (long long)r * row_vecs;
#pragma unroll
                    for (int v = 0; v < VPL; v++) {
                        const int c = lane + 32 * v;
                        buf[u][v] = FULLV ? ld_row16(row + c) : ld_row16_pred(row + c, c < nvec);
                    }
                }
#pragma unroll
                for (int u = 0; u < U; u++) {
#pragma unroll
                    for (int v = 0; v < VPL; v++) {
                        float f[EPV];
                        Elem<TableT>::unpack(buf[u][v], f);
#pragma unroll
                        for (int e = 0; e < EPV; e++) acc[v][e] = fmaf(ww[u], f[e], acc[v][e]);
                    }
                }
            }
        }

        // epilogue: + bias (one rounded add, as `outputs + self.bias`), convert, 16-byte stores
        OutT *orow = out + n * d + (long long)col0 * EPV;
#pragma unroll
        for (int v = 0; v < VPL; v++) {
            const int c = lane + 32 * v;
            if (c < nvec) {
                if (bias != nullptr) {
#pragma unroll
                    for (int e = 0; e < EPV; e++)
                        acc[v][e] = __fadd_rn(acc[v][e], __ldg(bias + (long long)(col0 + c) * EPV + e));
                }
                if constexpr (sizeof(OutT) == 4) {
#pragma unroll
                    for (int q = 0; q < EPV / 4; q++) {
                        float4 o = make_float4(acc[v][4 * q], acc[v][4 * q + 1], acc[v][4 * q + 2], acc[v][4 * q + 3]);
                        *reinterpret_cast<float4 *>(reinterpret_cast<float *>(orow) + c * EPV + 4 * q) = o;
                    }
                } else {
                    if constexpr (EPV == 8) {
                        uint4 o;
                        o.x = pack_bf16(acc[v][0], acc[v][1]);
                        o.y = pack_bf16(acc[v][2], acc[v][3]);
                        o.z = pack_bf16(acc[v][4], acc[v][5]);
                        o.w = pack_bf16(acc[v][6], acc[v][7]);
                        *reinterpret_cast<uint4 *>(reinterpret_cast<__nv_bfloat16 *>(orow) + c * 8) = o;
                    } else {
                        uint2 o;
                        o.x = pack_bf16(acc[v][0], acc[v][1]);
                        o.y = pack_bf16(acc[v][2], acc[v][3]);
                        *reinterpret_cast<uint2 *>(reinterpret_cast<__nv_bfloat16 *>(orow) + c * 4) = o;
                    }
                }
            }
        }
    }
    if (bad) atomicOr(status, LFFN_STATUS_INDEX_RANGE);
}

template <typename TableT, typename OutT, int VPL, bool FULLV>
static int launch_vpl_f(const int32_t *idx, const float *w, const void *tables, void *out, int64_t N, int I, int64_t S,
                      int d, int col0, const float *bias, const int2 *seg, cudaStream_t st) {
    constexpr int U = (VPL <= 3) ? LFFN_GATHER_U_NARROW : (VPL <= 6 ? LFFN_GATHER_U_MEDIUM : LFFN_GATHER_U_WIDE);
    constexpr int THREADS = LFFN_GATHER_THREADS;
    auto kern = gather_fwd_kernel<TableT, OutT, VPL, U, FULLV>;
    int per_sm = 0;
    LFFN_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, THREADS, 0));
    if (per_sm < 1) per_sm = 1;
    const long long want = (N + THREADS / 32 - 1) / (THREADS / 32);
    long long grid = (long long)num_sms() * per_sm;
    if (grid > want) grid = want;
    if (grid < 1) grid = 1;
    kern<<<(unsigned)grid, THREADS, 0, st>>>(idx, w, static_cast<const TableT *>(tables), static_cast<OutT *>(out), N, I,
                                             S, d, col0, bias, seg, status_word());
    LFFN_CHECK_CUDA(cudaGetLastError());
    return LFFN_OK;
}

// FULLV: the column tile is exactly VPL*32 vectors wide, so no lane needs a column predicate
template <typename TableT, typename OutT, int VPL>
static int launch_vpl(const int32_t *idx, const float *w, const void *tables, void *out, int64_t N, int I, int64_t S,
                      int d, int col0, const float *bias, const int2 *seg, cudaStream_t st) {
    const int nvec = min(d / Elem<TableT>::PER_VEC - col0, VPL * 32);
    if (nvec == VPL * 32)
        return launch_vpl_f<TableT, OutT, VPL, true>(idx, w, tables, out, N, I, S, d, col0, bias, seg, st);
    return launch_vpl_f<TableT, OutT, VPL, false>(idx, w, tables, out, N, I, S, d, col0, bias, seg, st);
}

template <typename TableT, typename OutT>
static int launch_typed(const int32_t *idx, const float *w, const void *tables, void *out, int64_t N, int I,
                        int64_t S, int d, const float *bias, const int2 *seg, cudaStream_t st) {
    constexpr int EPV = Elem<TableT>::PER_VEC;
    const int row_vecs = d / EPV;
    constexpr int MAXV = 8;  // widest column tile one launch covers: 8 vectors per lane
    for (int col0 = 0; col0 < row_vecs; col0 += MAXV * 32) {
        const int nvec = min(row_vecs - col0, MAXV * 32);
        const int vpl = (nvec + 31) / 32;
        int rc;
        switch (vpl) {
            case 1: rc = launch_vpl<TableT, OutT, 1>(idx, w, tables, out, N, I, S, d, col0, bias, seg, st); break;
            case 2: rc = launch_vpl<TableT, OutT, 2>(idx, w, tables, out, N, I, S, d, col0, bias, seg, st); break;
            case 3: rc = launch_vpl<TableT, OutT, 3>(idx, w, tables, out, N, I, S, d, col0, bias, seg, st); break;
            case 4: rc = launch_vpl<TableT, OutT, 4>(idx, w, tables, out, N, I, S, d, col0, bias, seg, st); break;
            case 5:
            case 6: rc = launch_vpl<TableT, OutT, 6>(idx, w, tables, out, N, I, S, d, col0, bias, seg, st); break;
            default: rc = launch_vpl<TableT, OutT, 8>(idx, w, tables, out, N, I, S, d, col0, bias, seg, st); break;
        }
        if (rc != LFFN_OK) return rc;
    }
    return LFFN_OK;
}

int launch_gather_fwd(const int32_t *idx, const float *w, const void *tables, int table_dtype, void *out,
                      int out_dtype, int64_t N, int I, int64_t S, int d, const float *bias, cudaStream_t st) {
    if (table_dtype == LFFN_F32 && out_dtype == LFFN_F32)
        return launch_typed<float, float>(idx, w, tables, out, N, I, S, d, bias, nullptr, st);
    if (table_dtype == LFFN_F32 && out_dtype == LFFN_BF16)
        return launch_typed<float, __nv_bfloat16>(idx, w, tables, out, N, I, S, d, bias, nullptr, st);
    if (table_dtype == LFFN_BF16 && out_dtype == LFFN_F32)
        return launch_typed<__nv_bfloat16, float>(idx, w, tables, out, N, I, S, d, bias, nullptr, st);
    if (table_dtype == LFFN_BF16 && out_dtype == LFFN_BF16)
        return launch_typed<__nv_bfloat16, __nv_bfloat16>(idx, w, tables, out, N, I, S, d, bias, nullptr, st);
    set_error("gather_fwd: unknown dtype (table %d, out %d)", table_dtype, out_dtype);
    return LFFN_ERR_INVALID_ARG;
}

// Segmented form used by the sorted table-gradient reduction: output row r sums the fp32 source rows
// src[idx[seg[r].x + j]] * w[seg[r].x + j], j < seg[r].y, in list order.
int launch_gather_segmented(const int32_t *idx, const float *w, const float *src, float *out, int64_t n_out,
                            const int2 *seg, int64_t n_src, int d, cudaStream_t st) {
    return launch_typed<float, float>(idx, w, src, out, n_out, 0, n_src, d, nullptr, seg, st);
}

}  // namespace lffn
