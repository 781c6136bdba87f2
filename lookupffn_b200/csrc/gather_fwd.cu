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

// values of `slab` below zero select how a row is added into the owner's buffer (lffn_gather_fwd_scatter); a slab
// index >= 0 may carry LFFN_SCATTER_SLAB_BULK:
constexpr int LFFN_SLAB_BULK_ADD = -1;    // one bulk reduction per row
constexpr int LFFN_SLAB_VECTOR_ADD = -2;  // 16-byte vector reductions

// 16-byte vector reduction into global memory, which may be another GPU's memory mapped over NVLink
__device__ __forceinline__ void red_add_v4_f32(float *p, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// SCATTER: instead of storing the row locally, send it to the rank that owns token n (n / rows_per_owner),
// peers[] holding every rank's buffer address (peer-mapped over NVLink): either added in place (vector
// reductions) or stored into this rank's slab of the owner's staging buffer.  Gather and the exchange step of the
// reduce-scatter become one kernel; the partial sums are never written to this GPU's HBM.
// SMODE: 0 = store the row locally; 1 / 2 / 3 / 4 = the scatter forms (bulk add, vector add, slab store with 16-byte
// stores, slab store as one bulk copy), one instantiation each so that every kernel carries only its own epilogue
template <typename TableT, typename OutT, int VPL, int U, bool FULLV, int SMODE = 0>
__global__ void __launch_bounds__(LFFN_GATHER_THREADS, LFFN_GATHER_MINBLOCKS) gather_fwd_kernel(const int32_t *__restrict__ idx, const float *__restrict__ w,
                                                         const TableT *__restrict__ tables, OutT *__restrict__ out,
                                                         long long N, int I, long long S, int d, int col0,
                                                         const float *__restrict__ bias, const int2 *__restrict__ seg,
                                                         int i0, int icnt, int resume, int finish, uint32_t *status,
                                                         float *const *__restrict__ peers, long long rows_per_owner,
                                                         int slab, long long rot, const OutT *residual) {
    constexpr bool SCATTER = SMODE != 0;
    // i0/icnt: the slice of each token's index list this launch consumes; resume: start from the fp32 partial
    // sums already in `out`; finish: last slice, add the bias and convert (see launch_vpl_f on why lists are sliced)
    // residual (may be null, may be `out` itself): [N, d] added after the bias, out = fl(fl(acc + bias) + residual),
    // the `dropout(FFN(x)) + x` of the encoder layer (layer.py:75-78) in inference
    constexpr int EPV = Elem<TableT>::PER_VEC;
    const int lane = threadIdx.x & 31;
    const int warps_per_block = blockDim.x >> 5;
    const long long warp0 = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * warps_per_block;
    const int row_vecs = d / EPV;              // 16-byte vectors per table row
    const int nvec = min(row_vecs - col0, VPL * 32);  // vectors this launch covers, starting at col0
    const uint4 *tv = reinterpret_cast<const uint4 *>(tables) + col0;
    bool bad = false;

    for (long long ni = warp0; ni < N; ni += nwarps) {
        // SCATTER: tokens are taken in rotated order (start at token `rot`), so that ranks running this kernel at
        // the same time, each with its own rotation, send to different owners at any moment
        const long long n = SCATTER ? (ni + rot >= N ? ni + rot - N : ni + rot) : ni;
        float acc[VPL][EPV];
#pragma unroll
        for (int v = 0; v < VPL; v++)
#pragma unroll
            for (int e = 0; e < EPV; e++) acc[v][e] = 0.f;
        if constexpr (sizeof(OutT) == 4) {
            if (resume) {  // continue the fmaf chains from the partial sums of the previous slice
                const float *prow = reinterpret_cast<const float *>(out) + n * d + (long long)col0 * EPV;
#pragma unroll
                for (int v = 0; v < VPL; v++) {
                    const int c = lane + 32 * v;
                    if (c < nvec) {
#pragma unroll
                        for (int q = 0; q < EPV / 4; q++) {
                            const float4 t = *reinterpret_cast<const float4 *>(prow + c * EPV + 4 * q);
                            acc[v][4 * q] = t.x;
                            acc[v][4 * q + 1] = t.y;
                            acc[v][4 * q + 2] = t.z;
                            acc[v][4 * q + 3] = t.w;
                        }
                    }
                }
            }
        }

        // dense [N, I] lists (slice [i0, i0+icnt) of each), or (segmented use: the sorted table-gradient
        // reduction) list n = seg[n].x .. +seg[n].y
        const int32_t *ip = idx + n * I + i0;
        const float *wp = w + n * I + i0;
        int In = icnt;
        if (seg != nullptr) {
            const int2 sg = __ldg(seg + n);
            ip = idx + sg.x;
            wp = w + sg.x;
            In = sg.y;
        }
        int my_i = 0;
        float my_w = 0.f;
        const unsigned long long pol_stream = policy_evict_first();
        if (lane < In) {
            my_i = ld_stream_i32(ip + lane, pol_stream);
            my_w = ld_stream_f32(wp + lane, pol_stream);
        }
        for (int g0 = 0; g0 < In; g0 += 32) {
            const int cur_i = my_i;
            const float cur_w = my_w;
            if (g0 + 32 + lane < In) {  // prefetch the next 32 (idx, w) pairs
                my_i = ld_stream_i32(ip + g0 + 32 + lane, pol_stream);
                my_w = ld_stream_f32(wp + g0 + 32 + lane, pol_stream);
            }
            const int cnt = min(32, In - g0);
            // The loop body is branch-free and free of per-row checks: every lane sanitises the one (index, weight)
            // pair it loaded -- an entry past the end of the list, or with an index outside [0, S), becomes (the
            // group's first row, weight 0); that row is part of the sum anyway, so the substitute adds exactly nothing
            // even when the row holds Inf or NaN -- and the loop only broadcasts sanitised pairs.
            int safe = __shfl_sync(FULL, cur_i, 0);
            safe = (unsigned long long)(long long)safe < (unsigned long long)S ? safe : 0;
            const bool mine_listed = lane < cnt;
            const bool mine_in_range = (unsigned long long)(long long)cur_i < (unsigned long long)S;
            bad |= mine_listed && !mine_in_range;
            const int san_i = (mine_listed && mine_in_range) ? cur_i : safe;
            const float san_w = (mine_listed && mine_in_range) ? cur_w : 0.f;
#pragma unroll 1
            for (int j0 = 0; j0 < cnt; j0 += U) {
                uint4 buf[U][VPL];
                float ww[U];
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int j = j0 + u;
                    const int r = __shfl_sync(FULL, san_i, j & 31);
                    const float wj = __shfl_sync(FULL, san_w, j & 31);
                    if constexpr (32 % U != 0) ww[u] = j < 32 ? wj : 0.f;  // a step that runs past lane 31 wraps around
                    else ww[u] = wj;
                    const uint4 *row = tv + (long long)r * row_vecs;
#pragma unroll
                    for (int v = 0; v < VPL; v++) {
                        const int c = lane + 32 * v;
                        buf[u][v] = FULLV ? ld_row16(row + c) : ld_row16_pred(row + c, c < nvec);
                    }
                }
                {
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
        }

        if constexpr (SCATTER) {
            // slab < 0: add into the owner's [rows_per_owner, d] buffer; slab >= 0: plain 16-byte stores into slab
            // `slab` of the owner's [n_ranks, rows_per_owner, d] staging buffer (the owner sums the slabs afterwards)
            const long long row = (slab < 0 ? 0 : (long long)slab * rows_per_owner) + n % rows_per_owner;
            float *prow = peers[n / rows_per_owner] + row * d + (long long)col0 * EPV;
            if constexpr (SMODE == 1 || SMODE == 4) {
                // One bulk transfer per row instead of 16-byte ones: the warp parks its fp32 row in shared memory and
                // lane 0 hands it to the TMA unit, which adds it into the owner's row (mode 1: cp.reduce.async.bulk,
                // f32 add) or stores it into this rank's slab of the owner's buffer (mode 4: cp.async.bulk) as one
                // transfer of up to 8 KB -- far fewer, larger packets on NVLink.
                extern __shared__ __align__(16) float stage_all[];
                float *stage = stage_all + (threadIdx.x >> 5) * (VPL * 32 * EPV);
                if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // previous row left smem
                __syncwarp();
#pragma unroll
                for (int v = 0; v < VPL; v++) {
                    const int c = lane + 32 * v;
                    if (c < nvec) {
#pragma unroll
                        for (int q = 0; q < EPV / 4; q++)
                            *reinterpret_cast<float4 *>(stage + c * EPV + 4 * q) =
                                make_float4(acc[v][4 * q], acc[v][4 * q + 1], acc[v][4 * q + 2], acc[v][4 * q + 3]);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the async proxy
                __syncwarp();
                if (lane == 0) {
                    const unsigned bytes = (unsigned)(nvec * EPV * sizeof(float));
                    if constexpr (SMODE == 1)
                        asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(
                                         __cvta_generic_to_global(prow)),
                                     "r"((unsigned)__cvta_generic_to_shared(stage)), "r"(bytes)
                                     : "memory");
                    else
                        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(
                                         __cvta_generic_to_global(prow)),
                                     "r"((unsigned)__cvta_generic_to_shared(stage)), "r"(bytes)
                                     : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
            } else {
#pragma unroll
                for (int v = 0; v < VPL; v++) {
                    const int c = lane + 32 * v;
                    if (c < nvec) {
#pragma unroll
                        for (int q = 0; q < EPV / 4; q++) {
                            if constexpr (SMODE == 2)
                                red_add_v4_f32(prow + c * EPV + 4 * q, acc[v][4 * q], acc[v][4 * q + 1], acc[v][4 * q + 2],
                                               acc[v][4 * q + 3]);
                            else
                                *reinterpret_cast<float4 *>(prow + c * EPV + 4 * q) =
                                    make_float4(acc[v][4 * q], acc[v][4 * q + 1], acc[v][4 * q + 2], acc[v][4 * q + 3]);
                        }
                    }
                }
            }
        } else {
            // epilogue: + bias (one rounded add, as `outputs + self.bias`), + residual, convert, 16-byte stores
            OutT *orow = out + n * d + (long long)col0 * EPV;
#pragma unroll
            for (int v = 0; v < VPL; v++) {
                const int c = lane + 32 * v;
                if (c < nvec) {
                    if (bias != nullptr && finish) {
#pragma unroll
                        for (int e = 0; e < EPV; e++)
                            acc[v][e] = __fadd_rn(acc[v][e], __ldg(bias + (long long)(col0 + c) * EPV + e));
                    }
                    if (residual != nullptr && finish) {
                        const OutT *rrow = residual + n * d + (long long)(col0 + c) * EPV;
#pragma unroll
                        for (int e = 0; e < EPV; e++) acc[v][e] = __fadd_rn(acc[v][e], Elem<OutT>::load1(rrow + e));
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
    }
    if constexpr (SCATTER) {
        // the bulk reductions of this thread have left shared memory and completed before the CTA exits
        if ((SMODE == 1 || SMODE == 4) && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
    if (bad) atomicOr(status, LFFN_STATUS_INDEX_RANGE);
}

template <typename TableT, typename OutT, int VPL, bool FULLV>
static int launch_vpl_f(const int32_t *idx, const float *w, const void *tables, void *out, int64_t N, int I, int64_t S,
                      int d, int col0, const float *bias, const int2 *seg, const void *residual, cudaStream_t st) {
    // rows in flight per warp; 2 KB bf16 rows (VPL = 4) measured best with 3 (config-5 shape: 2.41 -> 2.14 ms)
    constexpr int U = (VPL <= 3) ? LFFN_GATHER_U_NARROW
                      : (VPL == 4 && sizeof(TableT) == 2) ? 3
                      : (VPL <= 6 ? LFFN_GATHER_U_MEDIUM : LFFN_GATHER_U_WIDE);
    constexpr int THREADS = LFFN_GATHER_THREADS;
    auto kern = gather_fwd_kernel<TableT, OutT, VPL, U, FULLV>;
    int per_sm = 0;
    LFFN_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, THREADS, 0));
    if (per_sm < 1) per_sm = 1;
#ifdef LFFN_GATHER_CTAS_PER_SM
    if (per_sm > LFFN_GATHER_CTAS_PER_SM) per_sm = LFFN_GATHER_CTAS_PER_SM;  // tuning builds: leave room on the SM
#endif
    const long long want = (N + THREADS / 32 - 1) / (THREADS / 32);
    long long grid = (long long)num_sms() * per_sm;
    if (grid > want) grid = want;
    if (grid < 1) grid = 1;
    // Table sets well beyond L2 with long index lists (config 4: 403 MB of tables, 4608 entries per token): over
    // several waves of tokens the warps drift apart along the list, the band of tables being read outgrows L2 and
    // the kernel turns DRAM-bound.  Consuming the list in slices, one launch per slice over all tokens with the
    // fp32 partial sums parked in `out`, re-aligns the warps at every slice and keeps each launch's rows in L2
    // (measured 21.0 -> 12.8 ms on config 4).  The fmaf chains simply resume, so the result is bit-identical.
    // Only for fp32 outputs (a 16-bit output cannot hold the partial sums exactly) and dense lists.
    int slices = 1;
    if (sizeof(OutT) == 4 && seg == nullptr && I >= 512) {
        const double table_bytes = (double)S * d * sizeof(TableT);
        if (table_bytes > 256e6) slices = (int)(table_bytes / LFFN_GATHER_SLICE_BYTES);
        if (slices > I / 128) slices = I / 128;
        if (slices < 1) slices = 1;
    }
    if (residual == out) slices = 1;  // in-place residual: `out` cannot also park partial sums between slices
    const int per = slices == 1 ? I : ((I + slices - 1) / slices + 31) / 32 * 32;
    uint32_t *status = status_word();
    LFFN_REQUIRE(status != nullptr, LFFN_ERR_CUDA, "cannot locate the device status word");
    for (int i0 = 0; i0 == 0 || i0 < I; i0 += per) {
        const int icnt = I - i0 < per ? I - i0 : per;
        kern<<<(unsigned)grid, THREADS, 0, st>>>(idx, w, static_cast<const TableT *>(tables), static_cast<OutT *>(out), N,
                                                 I, S, d, col0, bias, seg, i0, icnt, i0 > 0 ? 1 : 0,
                                                 i0 + icnt >= I ? 1 : 0, status, nullptr, 0, -1, 0,
                                                 static_cast<const OutT *>(residual));
        LFFN_CHECK_CUDA(cudaGetLastError());
        if (I == 0) break;
    }
    return LFFN_OK;
}

template <typename TableT, int VPL, bool FULLV, int SMODE>
static int launch_scatter_f(const int32_t *idx, const float *w, const void *tables, float *const *peers,
                            long long rows_per_owner, int slab, long long rot, int64_t N, int I, int64_t S, int d, int col0,
                            cudaStream_t st) {
    // rows in flight per warp; 2 KB bf16 rows (VPL = 4) measured best with 3 (config-5 shape: 2.41 -> 2.14 ms)
    constexpr int U = (VPL <= 3) ? LFFN_GATHER_U_NARROW
                      : (VPL == 4 && sizeof(TableT) == 2) ? 3
                      : (VPL <= 6 ? LFFN_GATHER_U_MEDIUM : LFFN_GATHER_U_WIDE);
    constexpr int THREADS = LFFN_GATHER_THREADS;
    auto kern = gather_fwd_kernel<TableT, float, VPL, U, FULLV, SMODE>;
    int per_sm = 0;
    LFFN_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, THREADS, 0));
    if (per_sm < 1) per_sm = 1;
    const long long want = (N + THREADS / 32 - 1) / (THREADS / 32);
    long long grid = (long long)num_sms() * per_sm;
    if (grid > want) grid = want;
    if (grid < 1) grid = 1;
    uint32_t *status = status_word();
    LFFN_REQUIRE(status != nullptr, LFFN_ERR_CUDA, "cannot locate the device status word");
    const int slab_k = slab;
    const size_t smem = (SMODE == 1 || SMODE == 4) ? (size_t)(THREADS / 32) * VPL * 32 * Elem<TableT>::PER_VEC * sizeof(float) : 0;
    if (smem > 48 * 1024) LFFN_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    LFFN_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, THREADS, smem));
    if (per_sm < 1) per_sm = 1;
    grid = (long long)num_sms() * per_sm;
    if (grid > want) grid = want;
    if (grid < 1) grid = 1;
    kern<<<(unsigned)grid, THREADS, smem, st>>>(idx, w, static_cast<const TableT *>(tables), nullptr, N, I, S, d, col0, nullptr,
                                                nullptr, 0, I, 0, 1, status, peers, rows_per_owner, slab_k, rot, nullptr);
    LFFN_CHECK_CUDA(cudaGetLastError());
    return LFFN_OK;
}

template <typename TableT>
static int launch_scatter_typed(const int32_t *idx, const float *w, const void *tables, float *const *peers,
                                long long rows_per_owner, int slab, bool bulk_store, long long rot, int64_t N, int I, int64_t S,
                                int d, cudaStream_t st) {
    constexpr int EPV = Elem<TableT>::PER_VEC;
    const int row_vecs = d / EPV;
    constexpr int MAXV = 8;
    for (int col0 = 0; col0 < row_vecs; col0 += MAXV * 32) {
        const int nvec = min(row_vecs - col0, MAXV * 32);
        const int vpl = (nvec + 31) / 32;
        const bool full = nvec == vpl * 32;
        int rc;
#define LFFN_SCATTER_MODE(V, F)                                                                                              \
    (slab == LFFN_SLAB_BULK_ADD     ? launch_scatter_f<TableT, V, F, 1>(idx, w, tables, peers, rows_per_owner, slab, rot, N, I, S, d, col0, st) \
     : slab == LFFN_SLAB_VECTOR_ADD ? launch_scatter_f<TableT, V, F, 2>(idx, w, tables, peers, rows_per_owner, slab, rot, N, I, S, d, col0, st) \
     : bulk_store                   ? launch_scatter_f<TableT, V, F, 4>(idx, w, tables, peers, rows_per_owner, slab, rot, N, I, S, d, col0, st) \
                                    : launch_scatter_f<TableT, V, F, 3>(idx, w, tables, peers, rows_per_owner, slab, rot, N, I, S, d, col0, st))
#define LFFN_SCATTER_CASE(V) rc = full ? LFFN_SCATTER_MODE(V, true) : LFFN_SCATTER_MODE(V, false)
        switch (vpl) {
            case 1: LFFN_SCATTER_CASE(1); break;
            case 2: LFFN_SCATTER_CASE(2); break;
            case 3: LFFN_SCATTER_CASE(3); break;
            case 4: LFFN_SCATTER_CASE(4); break;
            case 5:
            case 6: LFFN_SCATTER_CASE(6); break;
            default: LFFN_SCATTER_CASE(8); break;
        }
#undef LFFN_SCATTER_CASE
#undef LFFN_SCATTER_MODE
        if (rc != LFFN_OK) return rc;
    }
    return LFFN_OK;
}

int launch_gather_fwd_scatter(const int32_t *idx, const float *w, const void *tables, int table_dtype,
                              float *const *peers, long long rows_per_owner, int slab, int first_owner, int64_t N, int I,
                              int64_t S, int d, cudaStream_t st) {
    const long long rot = N > 0 ? ((long long)first_owner * rows_per_owner) % N : 0;
    const bool bulk_store = slab >= 0 && (slab & LFFN_SCATTER_SLAB_BULK) != 0;
    if (slab >= 0) slab &= ~LFFN_SCATTER_SLAB_BULK;
    if (table_dtype == LFFN_F32)
        return launch_scatter_typed<float>(idx, w, tables, peers, rows_per_owner, slab, bulk_store, rot, N, I, S, d, st);
    if (table_dtype == LFFN_BF16)
        return launch_scatter_typed<__nv_bfloat16>(idx, w, tables, peers, rows_per_owner, slab, bulk_store, rot, N, I, S, d, st);
    set_error("gather_fwd_scatter: unknown table dtype %d", table_dtype);
    return LFFN_ERR_INVALID_ARG;
}

// FULLV: the column tile is exactly VPL*32 vectors wide, so no lane needs a column predicate
template <typename TableT, typename OutT, int VPL>
static int launch_vpl(const int32_t *idx, const float *w, const void *tables, void *out, int64_t N, int I, int64_t S,
                      int d, int col0, const float *bias, const int2 *seg, const void *residual, cudaStream_t st) {
    const int nvec = min(d / Elem<TableT>::PER_VEC - col0, VPL * 32);
    if (nvec == VPL * 32)
        return launch_vpl_f<TableT, OutT, VPL, true>(idx, w, tables, out, N, I, S, d, col0, bias, seg, residual, st);
    return launch_vpl_f<TableT, OutT, VPL, false>(idx, w, tables, out, N, I, S, d, col0, bias, seg, residual, st);
}

// maxv: the widest column tile one launch covers, in 16-byte vectors per lane (one of 1, 2, 3, 4, 6, 8)
template <typename TableT, typename OutT>
static int launch_typed(const int32_t *idx, const float *w, const void *tables, void *out, int64_t N, int I,
                        int64_t S, int d, const float *bias, const int2 *seg, const void *residual, cudaStream_t st,
                        int maxv = 8) {
    constexpr int EPV = Elem<TableT>::PER_VEC;
    const int row_vecs = d / EPV;
    const int MAXV = maxv;
    for (int col0 = 0; col0 < row_vecs; col0 += MAXV * 32) {
        const int nvec = min(row_vecs - col0, MAXV * 32);
        const int vpl = (nvec + 31) / 32;
        int rc;
        switch (vpl) {
            case 1: rc = launch_vpl<TableT, OutT, 1>(idx, w, tables, out, N, I, S, d, col0, bias, seg, residual, st); break;
            case 2: rc = launch_vpl<TableT, OutT, 2>(idx, w, tables, out, N, I, S, d, col0, bias, seg, residual, st); break;
            case 3: rc = launch_vpl<TableT, OutT, 3>(idx, w, tables, out, N, I, S, d, col0, bias, seg, residual, st); break;
            case 4: rc = launch_vpl<TableT, OutT, 4>(idx, w, tables, out, N, I, S, d, col0, bias, seg, residual, st); break;
            case 5:
            case 6: rc = launch_vpl<TableT, OutT, 6>(idx, w, tables, out, N, I, S, d, col0, bias, seg, residual, st); break;
            default: rc = launch_vpl<TableT, OutT, 8>(idx, w, tables, out, N, I, S, d, col0, bias, seg, residual, st); break;
        }
        if (rc != LFFN_OK) return rc;
    }
    return LFFN_OK;
}

int launch_gather_fwd(const int32_t *idx, const float *w, const void *tables, int table_dtype, void *out,
                      int out_dtype, int64_t N, int I, int64_t S, int d, const float *bias, const void *residual,
                      cudaStream_t st) {
    if (table_dtype == LFFN_F32 && out_dtype == LFFN_F32)
        return launch_typed<float, float>(idx, w, tables, out, N, I, S, d, bias, nullptr, residual, st);
    if (table_dtype == LFFN_F32 && out_dtype == LFFN_BF16)
        return launch_typed<float, __nv_bfloat16>(idx, w, tables, out, N, I, S, d, bias, nullptr, residual, st);
    if (table_dtype == LFFN_BF16 && out_dtype == LFFN_F32)
        return launch_typed<__nv_bfloat16, float>(idx, w, tables, out, N, I, S, d, bias, nullptr, residual, st);
    if (table_dtype == LFFN_BF16 && out_dtype == LFFN_BF16)
        return launch_typed<__nv_bfloat16, __nv_bfloat16>(idx, w, tables, out, N, I, S, d, bias, nullptr, residual, st);
    set_error("gather_fwd: unknown dtype (table %d, out %d)", table_dtype, out_dtype);
    return LFFN_ERR_INVALID_ARG;
}

// Segmented form used by the sorted table-gradient reduction: output row r sums the fp32 source rows
// src[idx[seg[r].x + j]] * w[seg[r].x + j], j < seg[r].y, in list order.
int launch_gather_segmented(const int32_t *idx, const float *w, const float *src, float *out, int64_t n_out,
                            const int2 *seg, int64_t n_src, int d, cudaStream_t st) {
    // The warps of this form do not stay aligned along the source rows (segments differ in length and every warp
    // restarts at row 0 with each new output row), so the whole source array is in use at any time.  Once it
    // outgrows what L2 keeps for data read from both dies, the rows are re-fetched from DRAM over and over (2.7 GB of
    // DRAM reads for a 67 MB source, L2 hit rate 57 %): narrower column tiles, one launch each, keep a tile's share
    // of the source resident instead.  The index lists are then read once per tile, which is small beside the rows.
    // Measured on a 50 MB source (16,384 x 768, 576 entries per output row): one launch 19.8 ms, tiles of 33 / 25 /
    // 17 / 8 MB 17.0 / 16.0 / 15.0 / 15.2 ms.
#ifndef LFFN_SEGMENTED_RESIDENT_BYTES
#define LFFN_SEGMENTED_RESIDENT_BYTES 20e6
#endif
    int maxv = 8;
    static const int widths[] = {8, 6, 4, 3, 2, 1};
    for (int i = 0; i < 6; i++) {
        maxv = widths[i];
        if ((double)n_src * maxv * 32 * 16 <= LFFN_SEGMENTED_RESIDENT_BYTES) break;
    }
    if (maxv * 32 > d / 4) maxv = 8;  // the row is narrower than the tile anyway: one launch
    return launch_typed<float, float>(idx, w, src, out, n_out, 0, n_src, d, nullptr, seg, nullptr, st, maxv);
}

}  // namespace lffn
