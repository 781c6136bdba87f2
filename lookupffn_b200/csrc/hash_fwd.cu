// Hashing stage: zero-pad -> R x S x (diagonal multiply, Walsh-Hadamard transform) -> mix ->
// bias -> sign-bit codes + gather weights.  Also the stand-alone transform and the
// codes/weights-from-z kernel.
//
// Replaces BH4.forward + bh4_cuda + compute_code_score_torch of the reference
// (lookup.py:29-39,64-77, bh4/kernel.py:23-36, compute_code_score/kernel.py:43-55) and its three
// Hadamard kernels (bh4/fast_hadamard_transform/extension/cuda_kernel.cu:19-257).
//
// Mapping (diagonal projection, BS = 1): one warp owns one token.  The D padded coordinates live
// in registers, V = D/32 per lane, coordinate e = j*32 + lane in register j.  Butterflies of
// stride >= 32 are register-register, strides 16..1 are warp shuffles; strides run from D/2
// down to 1 (the order of the reference's fp32 kernel, cuda_kernel.cu:234-252) and every
// butterfly is one rounded add and one rounded subtract, so sign bits reproduce on any
// implementation that keeps this order.  All R rotations of a token are done by the same warp:
// x is read from HBM once, nothing but codes and weights is written.
//
// Codes: for k in {1,2,4,8,16} one __ballot_sync per register packs 32 sign bits, i.e. 32/k
// codes, which lanes then cut out; other k (6, 10, 12: tables straddle registers and rotations)
// read the signs from the per-warp z buffer, with a 16-entry carry for a table that starts in
// the previous rotation.  Weights are accumulated serially over the k coordinates, as the
// reference's C++ does (compute_code_score/torch_extension.cc:30-40).
#include "common.cuh"
#include "hash_common.cuh"

namespace lffn {

// ---- Walsh-Hadamard transform in registers -----------------------------------------------------
template <int V>
__device__ __forceinline__ void fwht_regs(float (&v)[V], int lane) {
#pragma unroll
    for (int s = V / 2; s >= 1; s >>= 1) {  // strides 32*s: pairs of registers
#pragma unroll
        for (int j = 0; j < V; j++) {
            if ((j & s) == 0) {
                const float a = v[j], b = v[j + s];
                v[j] = __fadd_rn(a, b);
                v[j + s] = __fsub_rn(a, b);
            }
        }
    }
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) {  // strides 16..1: pairs of lanes
        const bool upper = (lane & s) != 0;
#pragma unroll
        for (int j = 0; j < V; j++) {
            const float p = __shfl_xor_sync(FULL, v[j], s);
            v[j] = upper ? __fsub_rn(p, v[j]) : __fadd_rn(v[j], p);
        }
    }
}

template <int V, typename XT>
__global__ void __launch_bounds__(256) fwht_kernel(const XT *__restrict__ x, XT *__restrict__ out, long long N,
                                                   float scale) {
    constexpr int D = V * 32;
    const int lane = threadIdx.x & 31;
    const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long n = warp0; n < N; n += nwarps) {
        float v[V];
        load_row<V, XT>(v, x + n * D, D, lane);
        fwht_regs<V>(v, lane);
#pragma unroll
        for (int j = 0; j < V; j++) {
            float o = v[j];
            if (scale != 1.f) o = __fmul_rn(o, scale);
            Elem<XT>::store1(out + n * D + j * 32 + lane, o);
        }
    }
}

// ---- the diagonal-projection hash kernel -------------------------------------------------------
constexpr int CARRY = 16;  // coordinates of the previous rotation kept for a straddling table
__host__ __device__ constexpr int zbuf_words(int D) { return CARRY + D + D / 32; }
__device__ __forceinline__ int zpad(int e) { return CARRY + e + (e >> 5); }

template <int V, typename XT>
__global__ void __launch_bounds__(128) hash_diag_kernel(HashArgs a) {
    constexpr int D = V * 32;
    extern __shared__ float smem[];
    const int lane = threadIdx.x & 31;
    const int wib = threadIdx.x >> 5;
    float *zs = smem + wib * (zbuf_words(D) + V);                          // z of the current rotation (+carry)
    unsigned *bits = reinterpret_cast<unsigned *>(zs + zbuf_words(D));     // V ballot words
    const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + wib;
    const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
    const int k = a.k;
    const int m = a.weight_mode == LFFN_WEIGHT_SOFT_FLIP ? k + 1 : 1;
    const bool use_ballot = (32 % k) == 0;
    const long long g_lo = (long long)a.t_begin * k, g_hi = (long long)(a.t_begin + a.t_count) * k;
    const long long out_pitch = (long long)a.t_count * m;

    for (long long n = warp0; n < a.N; n += nwarps) {
        const XT *xrow = static_cast<const XT *>(a.x) + n * a.d_in;
        float mean = 0.f, rstd = 1.f;
        if (a.ln_g != nullptr) {
            float v0[V];
            load_row<V, XT>(v0, xrow, a.d_in, lane);
            row_stats<V>(v0, a.d_in, lane, a.ln_eps, mean, rstd);
        }
        for (int r = a.r_lo; r <= a.r_hi; r++) {
            float v[V];
            load_row<V, XT>(v, xrow, a.d_in, lane);
            if (a.ln_g != nullptr) row_normalise<V>(v, a.d_in, lane, mean, rstd, a.ln_g, a.ln_b);
            for (int s = 0; s < a.S; s++) {
                const float *ws = a.w + ((long long)r * a.S + s) * D;
#pragma unroll
                for (int j = 0; j < V; j++) v[j] = __fmul_rn(v[j], __ldg(ws + j * 32 + lane));
                fwht_regs<V>(v, lane);
                if (a.had_scale != 1.f) {
#pragma unroll
                    for (int j = 0; j < V; j++) v[j] = __fmul_rn(v[j], a.had_scale);
                }
            }
            // z = fl(fl(mix_a * y) + fl(mix_b * u)) + bias
            float u[V];
            load_row<V, XT>(u, xrow, a.d_in, lane);
            if (a.ln_g != nullptr) row_normalise<V>(u, a.d_in, lane, mean, rstd, a.ln_g, a.ln_b);
            __syncwarp();  // every lane is done reading the previous rotation's buffer
            float keep = 0.f;
            if (lane < CARRY) keep = zs[zpad(D - CARRY + lane)];
            __syncwarp();
            if (lane < CARRY) zs[lane] = keep;
#pragma unroll
            for (int j = 0; j < V; j++) {
                const long long g = (long long)r * D + j * 32 + lane;
                float z = __fadd_rn(__fmul_rn(a.mix_a, v[j]), __fmul_rn(a.mix_b, u[j]));
                if (a.bias != nullptr && g < (long long)a.T * k) z = __fadd_rn(z, __ldg(a.bias + g));
                zs[zpad(j * 32 + lane)] = z;
                const unsigned b = __ballot_sync(FULL, z > 0.f);
                if (lane == 0) bits[j] = b;
                if (a.z_out != nullptr && g >= g_lo && g < g_hi) a.z_out[n * (g_hi - g_lo) + (g - g_lo)] = z;
            }
            __syncwarp();
            // tables that END inside this rotation: t*k + k <= (r+1)*D, and end after r*D
            const long long c_lo = (long long)r * D, c_hi = c_lo + D;
            long long t_first = c_lo / k;             // first table with end > c_lo
            if (t_first < a.t_begin) t_first = a.t_begin;
            long long t_end = c_hi / k;               // tables with end <= c_hi : t < c_hi / k
            if (t_end > a.t_begin + a.t_count) t_end = a.t_begin + a.t_count;
            if (a.idx_out == nullptr) t_end = t_first;  // projection only
            for (long long t = t_first + lane; t < t_end; t += 32) {
                const int local0 = (int)(t * k - c_lo);  // may be negative: starts in the previous rotation
                auto get = [&](int j) -> float {
                    const int e = local0 + j;
                    return e >= 0 ? zs[zpad(e)] : zs[CARRY + e];
                };
                bool have = false;
                int32_t code = 0;
                if (use_ballot) {  // local0 >= 0 and the k bits sit inside one ballot word
                    have = true;
                    code = (int32_t)((bits[local0 >> 5] >> (local0 & 31)) & ((1u << k) - 1u));
                }
                const long long o = n * out_pitch + (t - a.t_begin) * m;
                emit_table(get, k, a.bit_order, a.weight_mode, a.tau, (int32_t)((t - a.t_begin) << k), have, code,
                           a.idx_out + o, a.w_out + o);
            }
        }
        __syncwarp();
    }
}

// ---- the diagonal-projection hash kernel, vector layout ----------------------------------------------
// For D >= 256 and code lengths that divide 8.  Lane l holds NV = D/256 vectors of 8 consecutive
// coordinates: vector i covers e = (i*32 + l)*8 .. +7, so x, the diagonals and the bias are read with
// 16/32-byte loads and the k coordinates of a table (k | 8) sit in one lane: codes and weights are
// computed in registers, without shared memory, and consecutive lanes write consecutive tables.
// Butterfly order is unchanged (stride D/2 -> 1): vector index bits (register pairs), lane bits
// (shuffles; a +-1 multiplier turns the add/subtract choice into one fma, rounding as a plain
// add/subtract), then the three bits inside a vector (register pairs).
template <int NV>
__device__ __forceinline__ void fwht_vec8(float (&v)[NV][8], const float (&sgn)[5]) {
#pragma unroll
    for (int s = NV / 2; s >= 1; s >>= 1) {
#pragma unroll
        for (int i = 0; i < NV; i++) {
            if ((i & s) == 0) {
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    const float a = v[i][q], b = v[i + s][q];
                    v[i][q] = __fadd_rn(a, b);
                    v[i + s][q] = __fsub_rn(a, b);
                }
            }
        }
    }
#pragma unroll
    for (int b = 0; b < 5; b++) {
        const int s = 16 >> b;
#pragma unroll
        for (int i = 0; i < NV; i++) {
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const float p = __shfl_xor_sync(FULL, v[i][q], s);
                v[i][q] = __fmaf_rn(v[i][q], sgn[b], p);  // lower lane: v + p, upper lane: p - v
            }
        }
    }
#pragma unroll
    for (int s = 4; s >= 1; s >>= 1) {
#pragma unroll
        for (int i = 0; i < NV; i++) {
#pragma unroll
            for (int q = 0; q < 8; q++) {
                if ((q & s) == 0) {
                    const float a = v[i][q], b = v[i][q + s];
                    v[i][q] = __fadd_rn(a, b);
                    v[i][q + s] = __fsub_rn(a, b);
                }
            }
        }
    }
}

template <int NV, typename XT>
__device__ __forceinline__ void load_row_vec8(float (&v)[NV][8], const XT *row, int d_in, int lane, bool vec_ok) {
#pragma unroll
    for (int i = 0; i < NV; i++) {
        const int e0 = (i * 32 + lane) * 8;
        if (vec_ok && e0 + 8 <= d_in) {
            if constexpr (sizeof(XT) == 2) {
                const uint4 u = __ldg(reinterpret_cast<const uint4 *>(row + e0));
                Elem<__nv_bfloat16>::unpack(u, v[i]);
            } else {
                const float4 a = __ldg(reinterpret_cast<const float4 *>(row + e0));
                const float4 b = __ldg(reinterpret_cast<const float4 *>(row + e0 + 4));
                v[i][0] = a.x; v[i][1] = a.y; v[i][2] = a.z; v[i][3] = a.w;
                v[i][4] = b.x; v[i][5] = b.y; v[i][6] = b.z; v[i][7] = b.w;
            }
        } else {
#pragma unroll
            for (int q = 0; q < 8; q++) v[i][q] = (e0 + q < d_in) ? Elem<XT>::load1(row + e0 + q) : 0.f;
        }
    }
}

template <int NV>
__device__ __forceinline__ void row_stats_vec8(const float (&v)[NV][8], int d_in, int lane, float eps, float &mean,
                                               float &rstd) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; i++)
#pragma unroll
        for (int q = 0; q < 8; q++) s += v[i][q];
    mean = warp_sum(s) / (float)d_in;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < NV; i++)
#pragma unroll
        for (int q = 0; q < 8; q++) {
            const float c = ((i * 32 + lane) * 8 + q < d_in) ? v[i][q] - mean : 0.f;
            sq = fmaf(c, c, sq);
        }
    rstd = 1.f / sqrtf(warp_sum(sq) / (float)d_in + eps);
}

template <int NV>
__device__ __forceinline__ void row_normalise_vec8(float (&v)[NV][8], int d_in, int lane, float mean, float rstd,
                                                   const float *__restrict__ g, const float *__restrict__ b) {
#pragma unroll
    for (int i = 0; i < NV; i++)
#pragma unroll
        for (int q = 0; q < 8; q++) {
            const int e = (i * 32 + lane) * 8 + q;
            if (e < d_in) v[i][q] = ln_apply(v[i][q], mean, rstd, __ldg(g + e), b != nullptr ? __ldg(b + e) : 0.f);
        }
}

template <int NV, int K, typename XT>
__global__ void __launch_bounds__(128, (NV >= 8 ? 2 : 4)) hash_diag_vec8_kernel(HashArgs a, int x_vec_ok, int bias_vec_ok) {
    constexpr int D = NV * 256;
    const int lane = threadIdx.x & 31;
    const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
    constexpr int m_max = K + 1;
    const int m = a.weight_mode == LFFN_WEIGHT_SOFT_FLIP ? m_max : 1;
    const long long g_lo = (long long)a.t_begin * K, g_hi = (long long)(a.t_begin + a.t_count) * K;
    const long long out_pitch = (long long)a.t_count * m;
    float sgn[5];
#pragma unroll
    for (int b = 0; b < 5; b++) sgn[b] = (lane & (16 >> b)) ? -1.f : 1.f;

    for (long long n = warp0; n < a.N; n += nwarps) {
        const XT *xrow = static_cast<const XT *>(a.x) + n * a.d_in;
        float mean = 0.f, rstd = 1.f;
        if (a.ln_g != nullptr) {
            float v0[NV][8];
            load_row_vec8<NV, XT>(v0, xrow, a.d_in, lane, x_vec_ok != 0);
            row_stats_vec8<NV>(v0, a.d_in, lane, a.ln_eps, mean, rstd);
        }
        for (int r = a.r_lo; r <= a.r_hi; r++) {
            float v[NV][8];
            load_row_vec8<NV, XT>(v, xrow, a.d_in, lane, x_vec_ok != 0);
            if (a.ln_g != nullptr) row_normalise_vec8<NV>(v, a.d_in, lane, mean, rstd, a.ln_g, a.ln_b);
            for (int s = 0; s < a.S; s++) {
                const float *ws = a.w + ((long long)r * a.S + s) * D;
#pragma unroll
                for (int i = 0; i < NV; i++) {
                    const float4 w0 = __ldg(reinterpret_cast<const float4 *>(ws + (i * 32 + lane) * 8));
                    const float4 w1 = __ldg(reinterpret_cast<const float4 *>(ws + (i * 32 + lane) * 8 + 4));
                    v[i][0] = __fmul_rn(v[i][0], w0.x); v[i][1] = __fmul_rn(v[i][1], w0.y);
                    v[i][2] = __fmul_rn(v[i][2], w0.z); v[i][3] = __fmul_rn(v[i][3], w0.w);
                    v[i][4] = __fmul_rn(v[i][4], w1.x); v[i][5] = __fmul_rn(v[i][5], w1.y);
                    v[i][6] = __fmul_rn(v[i][6], w1.z); v[i][7] = __fmul_rn(v[i][7], w1.w);
                }
                fwht_vec8<NV>(v, sgn);
                if (a.had_scale != 1.f) {
#pragma unroll
                    for (int i = 0; i < NV; i++)
#pragma unroll
                        for (int q = 0; q < 8; q++) v[i][q] = __fmul_rn(v[i][q], a.had_scale);
                }
            }
            // z = fl(fl(mix_a * y) + fl(mix_b * u)) + bias; with mix_b == 0 the second term is +0
            if (a.mix_b != 0.f) {
                float u[NV][8];
                load_row_vec8<NV, XT>(u, xrow, a.d_in, lane, x_vec_ok != 0);
                if (a.ln_g != nullptr) row_normalise_vec8<NV>(u, a.d_in, lane, mean, rstd, a.ln_g, a.ln_b);
#pragma unroll
                for (int i = 0; i < NV; i++)
#pragma unroll
                    for (int q = 0; q < 8; q++)
                        v[i][q] = __fadd_rn(__fmul_rn(a.mix_a, v[i][q]), __fmul_rn(a.mix_b, u[i][q]));
            } else if (a.mix_a != 1.f) {
#pragma unroll
                for (int i = 0; i < NV; i++)
#pragma unroll
                    for (int q = 0; q < 8; q++) v[i][q] = __fmul_rn(a.mix_a, v[i][q]);
            }
#pragma unroll
            for (int i = 0; i < NV; i++) {
                const long long g0 = (long long)r * D + (i * 32 + lane) * 8;
                if (a.bias != nullptr && g0 < (long long)a.T * K) {
                    if (bias_vec_ok && g0 + 8 <= (long long)a.T * K) {
                        const float4 b0 = __ldg(reinterpret_cast<const float4 *>(a.bias + g0));
                        const float4 b1 = __ldg(reinterpret_cast<const float4 *>(a.bias + g0 + 4));
                        v[i][0] = __fadd_rn(v[i][0], b0.x); v[i][1] = __fadd_rn(v[i][1], b0.y);
                        v[i][2] = __fadd_rn(v[i][2], b0.z); v[i][3] = __fadd_rn(v[i][3], b0.w);
                        v[i][4] = __fadd_rn(v[i][4], b1.x); v[i][5] = __fadd_rn(v[i][5], b1.y);
                        v[i][6] = __fadd_rn(v[i][6], b1.z); v[i][7] = __fadd_rn(v[i][7], b1.w);
                    } else {
#pragma unroll
                        for (int q = 0; q < 8; q++)
                            if (g0 + q < (long long)a.T * K) v[i][q] = __fadd_rn(v[i][q], __ldg(a.bias + g0 + q));
                    }
                }
                if (a.z_out != nullptr) {
#pragma unroll
                    for (int q = 0; q < 8; q++) {
                        const long long g = g0 + q;
                        if (g >= g_lo && g < g_hi) a.z_out[n * (g_hi - g_lo) + (g - g_lo)] = v[i][q];
                    }
                }
                if (a.idx_out != nullptr) {
#pragma unroll
                    for (int sub = 0; sub < 8 / K; sub++) {
                        const long long t = g0 / K + sub;
                        if (t >= a.t_begin && t < a.t_begin + a.t_count) {
                            const long long o = n * out_pitch + (t - a.t_begin) * m;
                            emit_table_regs<K>(v[i], sub, a.bit_order, a.weight_mode, a.tau,
                                               (int32_t)((t - a.t_begin) << K), a.idx_out + o, a.w_out + o);
                        }
                    }
                }
            }
        }
    }
}

// ---- codes and weights from z in global memory (one thread per (token, table)) ------------------
__global__ void __launch_bounds__(256) code_weights_kernel(const float *__restrict__ z, long long NT, int T, int k,
                                                           int bit_order, int weight_mode, float tau, int add_offsets,
                                                           int32_t *__restrict__ idx_out, float *__restrict__ w_out) {
    const int m = weight_mode == LFFN_WEIGHT_SOFT_FLIP ? k + 1 : 1;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < NT; i += (long long)gridDim.x * blockDim.x) {
        const float *zp = z + i * k;
        auto get = [&](int j) -> float { return __ldg(zp + j); };
        const int t = (int)(i % T);
        emit_table(get, k, bit_order, weight_mode, tau, add_offsets ? (int32_t)(t << k) : 0, false, 0, idx_out + i * m,
                   w_out + i * m);
    }
}

// ---- gradient of the weights with respect to z (one thread per (token, table)) --------------------------
// score = num / den, num = sum_j a_j, den = prod_j (1 + e^{-2 a_j}), a = |z|:
//   d score / d z_j = sign(z_j) * (1 / den + score * 2 e^{-2 a_j} / (1 + e^{-2 a_j}))
// soft flip, w_c = prod_j f_cj with f = s_j or 1 - s_j, s = sigmoid(a / tau):
//   d w_c / d z_j = sign(z_j) / tau * w_c * (c == j+1 ? -s_j : 1 - s_j)
// sign(0) = 0, as torch.abs differentiates (compute_code_score/kernel.py:51-53 under autograd).
__global__ void __launch_bounds__(256) code_weights_bwd_kernel(const float *__restrict__ z, const float *__restrict__ dw,
                                                               long long NT, int k, int weight_mode, float tau,
                                                               float *__restrict__ dz) {
    const int m = weight_mode == LFFN_WEIGHT_SOFT_FLIP ? k + 1 : 1;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < NT; i += (long long)gridDim.x * blockDim.x) {
        const float *zp = z + i * k;
        float *dp = dz + i * k;
        if (weight_mode == LFFN_WEIGHT_ONES) {
            for (int j = 0; j < k; j++) dp[j] = 0.f;
        } else if (weight_mode == LFFN_WEIGHT_SCORE) {
            float num = 0.f, den = 1.f;
            for (int j = 0; j < k; j++) {
                const float a = fabsf(__ldg(zp + j));
                num += a;
                den *= 1.f + expf(-2.f * a);
            }
            const float score = num / den, g = __ldg(dw + i), inv_den = 1.f / den;
            for (int j = 0; j < k; j++) {
                const float zj = __ldg(zp + j), e = expf(-2.f * fabsf(zj));
                const float sg = zj > 0.f ? 1.f : (zj < 0.f ? -1.f : 0.f);
                dp[j] = g * sg * (inv_den + score * 2.f * e / (1.f + e));
            }
        } else {
            float s[16], acc[16];
            float hard = 1.f;
            for (int j = 0; j < k; j++) {
                s[j] = 1.f / (1.f + expf(-fabsf(__ldg(zp + j)) / tau));
                hard *= s[j];
                acc[j] = 0.f;
            }
            for (int c = 0; c <= k; c++) {
                float wc = 1.f;
                for (int j = 0; j < k; j++) wc *= (c == j + 1) ? (1.f - s[j]) : s[j];
                const float g = __ldg(dw + i * m + c) * wc;
                for (int j = 0; j < k; j++) acc[j] += g * ((c == j + 1) ? -s[j] : (1.f - s[j]));
            }
            for (int j = 0; j < k; j++) {
                const float zj = __ldg(zp + j);
                const float sg = zj > 0.f ? 1.f : (zj < 0.f ? -1.f : 0.f);
                dp[j] = sg * acc[j] / tau;
            }
            (void)hard;
        }
    }
}

// The reference's configuration (8-bit codes, score weights): a thread's table is two 16-byte loads and two 16-byte
// stores, and every exponential is evaluated once.  Same formulas as the general kernel above.
__global__ void __launch_bounds__(256) code_weights_bwd_score8_kernel(const float4 *__restrict__ z, const float *__restrict__ dw,
                                                                      long long NT, float4 *__restrict__ dz) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < NT; i += (long long)gridDim.x * blockDim.x) {
        const float4 lo = __ldg(z + 2 * i), hi = __ldg(z + 2 * i + 1);
        const float zz[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        float e[8], num = 0.f, den = 1.f;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float a = fabsf(zz[j]);
            e[j] = expf(-2.f * a);
            num += a;
            den *= 1.f + e[j];
        }
        const float score = num / den, g = __ldg(dw + i), inv_den = 1.f / den;
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float sg = zz[j] > 0.f ? 1.f : (zz[j] < 0.f ? -1.f : 0.f);
            o[j] = g * sg * (inv_den + score * 2.f * e[j] / (1.f + e[j]));
        }
        dz[2 * i] = make_float4(o[0], o[1], o[2], o[3]);
        dz[2 * i + 1] = make_float4(o[4], o[5], o[6], o[7]);
    }
}

int launch_code_weights_bwd(const float *z, const float *dw, int64_t N, int T, int k, int weight_mode, float tau,
                            float *dz, cudaStream_t st) {
    const long long NT = (long long)N * T;
    long long grid = (NT + 255) / 256;
    const long long cap = (long long)num_sms() * 8;
    if (grid > cap) grid = cap;
    if (grid < 1) grid = 1;
    if (k == 8 && weight_mode == LFFN_WEIGHT_SCORE && ((reinterpret_cast<uintptr_t>(z) | reinterpret_cast<uintptr_t>(dz)) & 15u) == 0) {
        code_weights_bwd_score8_kernel<<<(unsigned)grid, 256, 0, st>>>(reinterpret_cast<const float4 *>(z), dw, NT,
                                                                       reinterpret_cast<float4 *>(dz));
        LFFN_CHECK_CUDA(cudaGetLastError());
        return LFFN_OK;
    }
    code_weights_bwd_kernel<<<(unsigned)grid, 256, 0, st>>>(z, dw, NT, k, weight_mode, tau, dz);
    LFFN_CHECK_CUDA(cudaGetLastError());
    return LFFN_OK;
}

// ---- launchers -------------------------------------------------------------------------------
template <int V, typename XT>
static int launch_fwht_v(const void *x, void *out, int64_t N, float scale, cudaStream_t st) {
    const int threads = 256;
    long long grid = (N + 7) / 8;
    const long long cap = (long long)num_sms() * 8;
    if (grid > cap) grid = cap;
    if (grid < 1) grid = 1;
    fwht_kernel<V, XT><<<(unsigned)grid, threads, 0, st>>>(static_cast<const XT *>(x), static_cast<XT *>(out), N, scale);
    LFFN_CHECK_CUDA(cudaGetLastError());
    return LFFN_OK;
}

template <typename XT>
static int launch_fwht_t(const void *x, void *out, int64_t N, int D, float scale, cudaStream_t st) {
    switch (D) {
        case 32: return launch_fwht_v<1, XT>(x, out, N, scale, st);
        case 64: return launch_fwht_v<2, XT>(x, out, N, scale, st);
        case 128: return launch_fwht_v<4, XT>(x, out, N, scale, st);
        case 256: return launch_fwht_v<8, XT>(x, out, N, scale, st);
        case 512: return launch_fwht_v<16, XT>(x, out, N, scale, st);
        case 1024: return launch_fwht_v<32, XT>(x, out, N, scale, st);
        case 2048: return launch_fwht_v<64, XT>(x, out, N, scale, st);
    }
    set_error("fwht: D = %d is not a power of two in [32, 2048]", D);
    return LFFN_ERR_UNSUPPORTED;
}

int launch_fwht(const void *x, void *out, int64_t N, int D, int dtype, float scale, cudaStream_t st) {
    if (dtype == LFFN_F32) return launch_fwht_t<float>(x, out, N, D, scale, st);
    if (dtype == LFFN_BF16) return launch_fwht_t<__nv_bfloat16>(x, out, N, D, scale, st);
    set_error("fwht: unknown dtype %d", dtype);
    return LFFN_ERR_INVALID_ARG;
}

template <int V, typename XT>
static int launch_hash_diag_v(const HashArgs &a, cudaStream_t st) {
    constexpr int D = V * 32;
    constexpr int WARPS = 4;
    const size_t smem = (size_t)WARPS * (zbuf_words(D) + V) * sizeof(float);
    auto kern = hash_diag_kernel<V, XT>;
    LFFN_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int per_sm = 0;
    LFFN_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, WARPS * 32, smem));
    if (per_sm < 1) per_sm = 1;
    long long grid = (long long)num_sms() * per_sm;
    const long long want = (a.N + WARPS - 1) / WARPS;
    if (grid > want) grid = want;
    if (grid < 1) grid = 1;
    kern<<<(unsigned)grid, WARPS * 32, smem, st>>>(a);
    LFFN_CHECK_CUDA(cudaGetLastError());
    return LFFN_OK;
}

template <int NV, int K, typename XT>
static int launch_hash_vec8_nk(const HashArgs &a, cudaStream_t st) {
    constexpr int WARPS = 4;
    auto kern = hash_diag_vec8_kernel<NV, K, XT>;
    int per_sm = 0;
    LFFN_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, WARPS * 32, 0));
    if (per_sm < 1) per_sm = 1;
    long long grid = (long long)num_sms() * per_sm;
    const long long want = (a.N + WARPS - 1) / WARPS;
    if (grid > want) grid = want;
    if (grid < 1) grid = 1;
    const size_t esz = sizeof(XT);
    const int x_vec_ok = ((a.d_in * esz) % 16 == 0) && ((reinterpret_cast<uintptr_t>(a.x) & 15u) == 0);
    const int bias_vec_ok = a.bias != nullptr && (reinterpret_cast<uintptr_t>(a.bias) & 15u) == 0;
    kern<<<(unsigned)grid, WARPS * 32, 0, st>>>(a, x_vec_ok, bias_vec_ok);
    LFFN_CHECK_CUDA(cudaGetLastError());
    return LFFN_OK;
}

template <int NV, typename XT>
static int launch_hash_vec8_n(const HashArgs &a, cudaStream_t st) {
    switch (a.k) {
        case 1: return launch_hash_vec8_nk<NV, 1, XT>(a, st);
        case 2: return launch_hash_vec8_nk<NV, 2, XT>(a, st);
        case 4: return launch_hash_vec8_nk<NV, 4, XT>(a, st);
        default: return launch_hash_vec8_nk<NV, 8, XT>(a, st);
    }
}

template <typename XT>
static int launch_hash_diag_t(const HashArgs &a, cudaStream_t st) {
    int rc_t = LFFN_OK;
    if (try_launch_hash_transposing(a, sizeof(XT) == 2 ? LFFN_BF16 : LFFN_F32, st, &rc_t)) return rc_t;
    const bool w_aligned = (reinterpret_cast<uintptr_t>(a.w) & 15u) == 0;
    if (w_aligned && (a.k == 1 || a.k == 2 || a.k == 4 || a.k == 8)) {  // vector layout
        switch (a.D) {
            case 256: return launch_hash_vec8_n<1, XT>(a, st);
            case 512: return launch_hash_vec8_n<2, XT>(a, st);
            case 1024: return launch_hash_vec8_n<4, XT>(a, st);
            case 2048: return launch_hash_vec8_n<8, XT>(a, st);
        }
    }
    switch (a.D) {
        case 64: return launch_hash_diag_v<2, XT>(a, st);
        case 128: return launch_hash_diag_v<4, XT>(a, st);
        case 256: return launch_hash_diag_v<8, XT>(a, st);
        case 512: return launch_hash_diag_v<16, XT>(a, st);
        case 1024: return launch_hash_diag_v<32, XT>(a, st);
        case 2048: return launch_hash_diag_v<64, XT>(a, st);
    }
    set_error("hash_fwd: D = %d is not a power of two in [64, 2048]", a.D);
    return LFFN_ERR_UNSUPPORTED;
}

int launch_hash_block(const HashArgs &a, int BS, int transpose_w, int x_dtype, cudaStream_t st);  // hash_block.cu

int launch_hash_fwd(const lffn_hash_desc &h, const void *x, int x_dtype, int64_t N, int t_begin, int t_count,
                    int32_t *idx_out, float *w_out, float *z_out, const float *ln_g, const float *ln_b, float ln_eps,
                    cudaStream_t st) {
    HashArgs a;
    a.act_out = nullptr;
    a.dz = nullptr;
    a.dz_cols = 0;
    a.du_out = nullptr;
    a.ln_g = ln_g;
    a.ln_b = ln_b;
    a.ln_eps = ln_eps;
    a.x = x;
    a.N = N;
    a.d_in = h.d_in;
    a.D = h.D;
    a.S = h.S;
    a.R = h.R;
    a.r_lo = (int)(((long long)t_begin * h.k) / h.D);
    a.r_hi = (int)(((long long)(t_begin + t_count) * h.k - 1) / h.D);
    a.had_scale = h.had_scale;
    a.mix_a = h.mix_a;
    a.mix_b = h.mix_b;
    a.w = h.proj_w;
    a.bias = h.proj_bias;
    a.T = h.T;
    a.k = h.k;
    a.bit_order = h.bit_order;
    a.weight_mode = h.weight_mode;
    a.tau = h.tau;
    a.t_begin = t_begin;
    a.t_count = t_count;
    a.idx_out = idx_out;
    a.w_out = w_out;
    a.z_out = z_out;
    a.status = status_word();
    if (h.BS == 1) {
        if (x_dtype == LFFN_F32) return launch_hash_diag_t<float>(a, st);
        if (x_dtype == LFFN_BF16) return launch_hash_diag_t<__nv_bfloat16>(a, st);
        set_error("hash_fwd: unknown x dtype %d", x_dtype);
        return LFFN_ERR_INVALID_ARG;
    }
    return launch_hash_block(a, h.BS, h.transpose_w, x_dtype, st);
}

int launch_code_weights(const float *z, int64_t N, int T, int k, int bit_order, int weight_mode, float tau,
                        int add_offsets, int32_t *idx_out, float *w_out, cudaStream_t st) {
    const long long NT = (long long)N * T;
    long long grid = (NT + 255) / 256;
    const long long cap = (long long)num_sms() * 8;
    if (grid > cap) grid = cap;
    if (grid < 1) grid = 1;
    code_weights_kernel<<<(unsigned)grid, 256, 0, st>>>(z, NT, T, k, bit_order, weight_mode, tau, add_offsets, idx_out,
                                                        w_out);
    LFFN_CHECK_CUDA(cudaGetLastError());
    return LFFN_OK;
}

}  // namespace lffn
