// Hashing stage, diagonal projection, transposing layout: the kernel that serves codes-and-weights requests of the
// common shapes (see hash_fwd.cu for the other layouts and for what the stage computes).
#include "common.cuh"
#include "hash_common.cuh"

namespace lffn {

// ---- the diagonal-projection hash kernel, transposing layout -----------------------------------------------
// For D in {256, 512, 1024}, no z output and no mix with the input (mix_b == 0); any code length (those that divide
// D/32 keep a lane's tables in registers, the others read the finished rotation back from the warp's buffer).
// A transform of D = 32 V points needs log2(D) butterfly stages over 5 lane bits and log2(V) register bits; instead
// of paying a shuffle per value for every lane-bit stage, the warp changes layout in the middle of each transform
// through a padded per-warp shared-memory buffer:
//   layout A: lane = e & 31, register j = e >> 5       (coalesced loads of x and of the diagonals)
//             stages of stride D/2 .. 32 are register pairs; the 5 - log2(V) stages of stride 16 .. V are shuffles
//   layout B: lane = e / V, register c = e % V         (a lane holds V consecutive coordinates)
//             stages of stride V/2 .. 1 are register pairs; the V/K tables of a lane have their K coordinates in
//             registers, and consecutive lanes write consecutive groups of tables with 16-byte stores
// The stage order is still stride D/2 down to 1 and every butterfly one rounded add and one rounded subtract, so z
// is bit-identical to the other layouts and to the CPU oracle.  Buffer address of coordinate e: e + 4 (e >> 5);
// with it the 32-bit accesses of layout A and the 128-bit accesses of layout B are both free of bank conflicts.
// x is read once per token and kept in registers (layout A) for all rotations; the optional LayerNorm is applied to
// those registers.  The projection bias, which must be added in layout B, is staged once per CTA in shared memory
// in the buffer's address order.
__device__ __forceinline__ int tbuf_addr(int e) { return e + ((e >> 5) << 2); }
__host__ __device__ constexpr int tbuf_words(int D) { return D + D / 8; }

template <int V>
__device__ __forceinline__ void regs_to_layout_b(float (&v)[V], float *buf, int lane) {
#pragma unroll
    for (int j = 0; j < V; j++) buf[j * 36 + lane] = v[j];  // tbuf_addr(j * 32 + lane)
    __syncwarp();
#pragma unroll
    for (int q = 0; q < V / 4; q++) {
        const float4 t = *reinterpret_cast<const float4 *>(buf + tbuf_addr(lane * V + 4 * q));
        v[4 * q] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
    }
    __syncwarp();
}

template <int V>
__device__ __forceinline__ void regs_to_layout_a(float (&v)[V], float *buf, int lane) {
#pragma unroll
    for (int q = 0; q < V / 4; q++)
        *reinterpret_cast<float4 *>(buf + tbuf_addr(lane * V + 4 * q)) =
            make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    __syncwarp();
#pragma unroll
    for (int j = 0; j < V; j++) v[j] = buf[j * 36 + lane];
    __syncwarp();
}

// one transform: in layout A on entry, in layout B on exit
template <int V>
__device__ __forceinline__ void fwht_a_to_b(float (&v)[V], float *buf, int lane) {
    reg_butterflies<V>(v);  // strides 32 s, s = V/2 .. 1
#pragma unroll
    for (int s = 16; s >= V; s >>= 1) {  // strides 16 .. V (none for V = 32): lane pairs
        const float sg = (lane & s) ? -1.f : 1.f;
#pragma unroll
        for (int j = 0; j < V; j += 2) {
            const float p0 = __shfl_xor_sync(FULL, v[j], s), p1 = __shfl_xor_sync(FULL, v[j + 1], s);
            fma2(v[j], v[j + 1], v[j], v[j + 1], sg, sg, p0, p1);  // lower lane: v + p, upper lane: p - v
        }
    }
    regs_to_layout_b<V>(v, buf, lane);
    reg_butterflies<V>(v);  // strides V/2 .. 1
}

constexpr int HT_WARPS = 4;
constexpr int HT_CARRY = 16;  // coordinates of the previous rotation kept for a straddling table (k <= 16)

template <int V, int K, typename XT>
__global__ void __launch_bounds__(HT_WARPS * 32, 4) hash_diag_t_kernel(HashArgs a) {
    // K = 0: any code length (a.k), tables may straddle lanes and rotations -- the finished rotation goes back to the
    // warp's buffer and lanes stride over the tables that end in it (HT_CARRY coordinates of the previous rotation
    // are kept for a table that began there); K > 0: K divides V and a lane's tables sit in its registers.
    constexpr int D = V * 32;
    constexpr int KK = K > 0 ? K : 1;
    constexpr int TPL = V / KK;  // tables per lane per rotation (K > 0)
    extern __shared__ __align__(16) float smem_t[];
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    float *buf = smem_t + wib * (tbuf_words(D) + HT_CARRY);
    float *carry = buf + tbuf_words(D);
    float *sbias = smem_t + HT_WARPS * (tbuf_words(D) + HT_CARRY);  // [r_hi - r_lo + 1][tbuf_words(D)] when a.bias != nullptr
    // second per-warp buffer behind the staged bias, only for the soft-flip mode with K >= 8 (see the emission below)
    float *stage2 = nullptr;
    if (K >= 8 && a.weight_mode == LFFN_WEIGHT_SOFT_FLIP && (reinterpret_cast<uintptr_t>(a.idx_out) & 15u) == 0 &&
        (reinterpret_cast<uintptr_t>(a.w_out) & 15u) == 0 && (((long long)a.t_count * (K + 1)) & 3) == 0)
        stage2 = sbias + (a.bias != nullptr ? (a.r_hi - a.r_lo + 1) * tbuf_words(D) : 0) + wib * tbuf_words(D);
    const int k = K > 0 ? K : a.k;
    const long long total = (long long)a.T * k;
    if (a.bias != nullptr) {
        const int nrot = a.r_hi - a.r_lo + 1;
        for (int i = threadIdx.x; i < nrot * D; i += blockDim.x) {
            const int rr = i / D, e = i - rr * D;
            const long long g = (long long)(a.r_lo + rr) * D + e;
            sbias[rr * tbuf_words(D) + tbuf_addr(e)] = g < total ? __ldg(a.bias + g) : 0.f;
        }
        __syncthreads();
    }
    const long long warp0 = (long long)blockIdx.x * HT_WARPS + wib;
    const long long nwarps = (long long)gridDim.x * HT_WARPS;
    const int m = a.weight_mode == LFFN_WEIGHT_SOFT_FLIP ? k + 1 : 1;
    const long long out_pitch = (long long)a.t_count * m;
    // one 16-byte store per four tables needs m == 1, aligned output rows and four tables per group
    const bool vec4 = K > 0 && m == 1 && (TPL % 4 == 0) && (out_pitch & 3) == 0 && (a.t_begin & 3) == 0 &&
                      ((reinterpret_cast<uintptr_t>(a.idx_out) & 15u) == 0) && ((reinterpret_cast<uintptr_t>(a.w_out) & 15u) == 0);

    for (long long n = warp0; n < a.N; n += nwarps) {
        const XT *xrow = static_cast<const XT *>(a.x) + n * a.d_in;
        float xr[V];
        load_row<V, XT>(xr, xrow, a.d_in, lane);
        if (a.ln_g != nullptr) {
            float mean, rstd;
            row_stats<V>(xr, a.d_in, lane, a.ln_eps, mean, rstd);
            row_normalise<V>(xr, a.d_in, lane, mean, rstd, a.ln_g, a.ln_b);
        }
        for (int r = a.r_lo; r <= a.r_hi; r++) {
            float v[V];
            for (int s = 0; s < a.S; s++) {
                const float *ws = a.w + ((long long)r * a.S + s) * D;
                // the products below feed the butterflies' adds: scalar multiplies (see the rule beside mul2)
                if (s == 0) {
#pragma unroll
                    for (int j = 0; j < V; j++) v[j] = __fmul_rn(xr[j], __ldg(ws + j * 32 + lane));
                } else {
                    regs_to_layout_a<V>(v, buf, lane);
#pragma unroll
                    for (int j = 0; j < V; j++) v[j] = __fmul_rn(v[j], __ldg(ws + j * 32 + lane));
                }
                fwht_a_to_b<V>(v, buf, lane);
                if (a.had_scale != 1.f) {
                    if (s + 1 < a.S) {  // followed by the next diagonal's multiply: packed
#pragma unroll
                        for (int c = 0; c < V; c += 2) mul2(v[c], v[c + 1], v[c], v[c + 1], a.had_scale, a.had_scale);
                    } else {            // followed by the bias add: scalar
#pragma unroll
                        for (int c = 0; c < V; c++) v[c] = __fmul_rn(v[c], a.had_scale);
                    }
                }
            }
            // layout B: v[c] is coordinate r * D + lane * V + c.  z = fl(mix_a * y) (+ 0) + bias
            if (a.mix_a != 1.f) {
#pragma unroll
                for (int c = 0; c < V; c++) v[c] = __fmul_rn(a.mix_a, v[c]);
            }
            if (a.bias != nullptr) {
                const float *sb = sbias + (r - a.r_lo) * tbuf_words(D);
#pragma unroll
                for (int q = 0; q < V / 4; q++) {
                    const float4 b = *reinterpret_cast<const float4 *>(sb + tbuf_addr(lane * V + 4 * q));
                    add2(v[4 * q], v[4 * q + 1], v[4 * q], v[4 * q + 1], b.x, b.y);
                    add2(v[4 * q + 2], v[4 * q + 3], v[4 * q + 2], v[4 * q + 3], b.z, b.w);
                }
            }
            if constexpr (K == 0) {
                // back to the buffer (coordinate e of this rotation at tbuf_addr(e)), then one table per lane at a time
                // (carry[] holds the tail of the previous rotation, saved below before the buffer was reused)
                __syncwarp();
#pragma unroll
                for (int q = 0; q < V / 4; q++)
                    *reinterpret_cast<float4 *>(buf + tbuf_addr(lane * V + 4 * q)) =
                        make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                __syncwarp();
                const long long c_lo = (long long)r * D, c_hi = c_lo + D;
                long long t_first = c_lo / k;  // first table that ends after c_lo
                if (t_first < a.t_begin) t_first = a.t_begin;
                long long t_end = c_hi / k;    // tables that end at or before c_hi
                if (t_end > a.t_begin + a.t_count) t_end = a.t_begin + a.t_count;
                for (long long t = t_first + lane; t < t_end; t += 32) {
                    const int local0 = (int)(t * k - c_lo);  // negative: the table began in the previous rotation
                    auto get = [&](int j) -> float {
                        const int e = local0 + j;
                        return e >= 0 ? buf[tbuf_addr(e)] : carry[HT_CARRY + e];
                    };
                    const long long o = n * out_pitch + (t - a.t_begin) * m;
                    emit_table(get, k, a.bit_order, a.weight_mode, a.tau, (int32_t)((t - a.t_begin) << k), false, 0,
                               a.idx_out + o, a.w_out + o);
                }
                __syncwarp();
                if (lane < HT_CARRY) carry[lane] = buf[tbuf_addr(D - HT_CARRY + lane)];  // this rotation's tail
                __syncwarp();
                continue;
            }
            const long long t0 = ((long long)r * D + lane * V) / KK;  // first table of this lane in this rotation
            if constexpr (K >= 8) {
                // k + 1 candidates per table (soft flip): the rotation's D/K tables x (K + 1) pairs are collected in
                // two per-warp buffers and leave as 16-byte stores of consecutive lanes, instead of 4-byte stores
                // 36 (K + 1) bytes apart
                constexpr int E = (D / KK) * (KK + 1);  // pairs per rotation; <= tbuf_words(D) for K >= 8
                const long long tr0 = (long long)r * D / KK;
                const long long o0 = n * out_pitch + (tr0 - a.t_begin) * m;
                if (stage2 != nullptr && tr0 >= a.t_begin && tr0 + D / KK <= a.t_begin + a.t_count && (o0 & 3) == 0) {
                    int32_t *ib = reinterpret_cast<int32_t *>(buf);
                    float *wb = stage2;
#pragma unroll
                    for (int u = 0; u < TPL; u++)
                        emit_table_k<KK>(&v[u * KK], a.bit_order, a.weight_mode, a.tau, (int32_t)((t0 + u - a.t_begin) << KK),
                                        ib + (lane * TPL + u) * (KK + 1), wb + (lane * TPL + u) * (KK + 1));
                    __syncwarp();
                    for (int i = lane; i < E / 4; i += 32) {
                        reinterpret_cast<int4 *>(a.idx_out + o0)[i] = reinterpret_cast<const int4 *>(ib)[i];
                        reinterpret_cast<float4 *>(a.w_out + o0)[i] = reinterpret_cast<const float4 *>(wb)[i];
                    }
                    __syncwarp();
                    continue;
                }
            }
            if (vec4) {
#pragma unroll
                for (int g4 = 0; g4 < TPL / 4; g4++) {
                    const long long t = t0 + 4 * g4;
                    if (t >= a.t_begin && t + 4 <= a.t_begin + a.t_count) {
                        int32_t ci[4];
                        float cw[4];
#pragma unroll
                        for (int u = 0; u < 4; u++)
                            emit_table_k<KK>(&v[(4 * g4 + u) * KK], a.bit_order, a.weight_mode, a.tau,
                                            (int32_t)((t + u - a.t_begin) << KK), ci + u, cw + u);
                        const long long o = n * out_pitch + (t - a.t_begin);
                        *reinterpret_cast<int4 *>(a.idx_out + o) = make_int4(ci[0], ci[1], ci[2], ci[3]);
                        *reinterpret_cast<float4 *>(a.w_out + o) = make_float4(cw[0], cw[1], cw[2], cw[3]);
                    } else {
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const long long tt = t + u;
                            if (tt >= a.t_begin && tt < a.t_begin + a.t_count) {
                                const long long o = n * out_pitch + (tt - a.t_begin);
                                emit_table_k<KK>(&v[(4 * g4 + u) * KK], a.bit_order, a.weight_mode, a.tau,
                                                (int32_t)((tt - a.t_begin) << KK), a.idx_out + o, a.w_out + o);
                            }
                        }
                    }
                }
            } else {
#pragma unroll
                for (int u = 0; u < TPL; u++) {
                    const long long tt = t0 + u;
                    if (tt >= a.t_begin && tt < a.t_begin + a.t_count) {
                        const long long o = n * out_pitch + (tt - a.t_begin) * m;
                        emit_table_k<KK>(&v[u * KK], a.bit_order, a.weight_mode, a.tau, (int32_t)((tt - a.t_begin) << KK),
                                        a.idx_out + o, a.w_out + o);
                    }
                }
            }
        }
    }
}

template <int V, int K, typename XT>
static int launch_hash_t_vk(const HashArgs &a, size_t smem, cudaStream_t st) {
    auto kern = hash_diag_t_kernel<V, K, XT>;
    if (smem > 48 * 1024) LFFN_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int per_sm = 0;
    LFFN_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, HT_WARPS * 32, smem));
    if (per_sm < 1) per_sm = 1;
    long long grid = (long long)num_sms() * per_sm;
    const long long want = (a.N + HT_WARPS - 1) / HT_WARPS;
    if (grid > want) grid = want;
    if (grid < 1) grid = 1;
    kern<<<(unsigned)grid, HT_WARPS * 32, smem, st>>>(a);
    LFFN_CHECK_CUDA(cudaGetLastError());
    return LFFN_OK;
}

template <int V, typename XT>
static int launch_hash_t_v(const HashArgs &a, size_t smem, cudaStream_t st) {
    switch (a.k) {
        case 1: return launch_hash_t_vk<V, 1, XT>(a, smem, st);
        case 2: return launch_hash_t_vk<V, 2, XT>(a, smem, st);
        case 4: return launch_hash_t_vk<V, 4, XT>(a, smem, st);
        case 8: return launch_hash_t_vk<V, 8, XT>(a, smem, st);
    }
    if constexpr (V >= 16) {
        if (a.k == 16) return launch_hash_t_vk<V, 16, XT>(a, smem, st);
    }
    return launch_hash_t_vk<V, 0, XT>(a, smem, st);  // any other code length up to 16
}

// The transposing layout covers codes-and-weights requests (no z output) without the input mix, D = 256 .. 1024,
// k dividing D / 32, and a projection bias small enough to stage in shared memory.  Returns false when it does not apply.
template <typename XT>
static bool try_launch_hash_t(const HashArgs &a, cudaStream_t st, int *rc) {
#ifdef LFFN_HASH_NO_TRANSPOSING_LAYOUT
    return false;
#endif
    if (a.z_out != nullptr || a.idx_out == nullptr || a.mix_b != 0.f) return false;
    if (a.D != 256 && a.D != 512 && a.D != 1024) return false;
    if (a.k < 1 || a.k > 16) return false;
    const size_t nrot = (size_t)(a.r_hi - a.r_lo + 1);
    size_t smem = ((size_t)HT_WARPS * (tbuf_words(a.D) + HT_CARRY) + (a.bias != nullptr ? nrot : 0) * tbuf_words(a.D)) * sizeof(float);
    if (smem > 40 * 1024) return false;
    if (a.weight_mode == LFFN_WEIGHT_SOFT_FLIP && (a.k == 8 || a.k == 16))  // the second staging buffer per warp
        smem += (size_t)HT_WARPS * tbuf_words(a.D) * sizeof(float);
    switch (a.D) {
        case 256: *rc = launch_hash_t_v<8, XT>(a, smem, st); break;
        case 512: *rc = launch_hash_t_v<16, XT>(a, smem, st); break;
        default: *rc = launch_hash_t_v<32, XT>(a, smem, st); break;
    }
    return true;
}

bool try_launch_hash_transposing(const HashArgs &a, int x_dtype, cudaStream_t st, int *rc) {
    if (x_dtype == LFFN_F32) return try_launch_hash_t<float>(a, st, rc);
    if (x_dtype == LFFN_BF16) return try_launch_hash_t<__nv_bfloat16>(a, st, rc);
    return false;
}

}  // namespace lffn
