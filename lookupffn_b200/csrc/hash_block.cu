// Hashing stage with block-diagonal projection weights (BS >= 4): the reference's BH4
// (lookup.py:10-47, bh4/kernel.py:23-36): R x S x (block-diagonal multiply, Hadamard), mix,
// bias, then codes and weights (compute_code_score/kernel.py:43-55).
//
// Mapping: one CTA of 256 threads owns a tile of M = 32 tokens for all rotations and stages; the
// tile lives in shared memory TRANSPOSED, Y[e][m] (coordinate-major, tokens contiguous, row
// padded to 36 floats), so that
//   - the block multiply reads 8 tokens of one input coordinate as two 16-byte broadcasts and 4
//     output columns of the staged weights as one 16-byte load, for an 8 x 4 register tile
//     per thread (32 fused multiply-adds per 3 shared loads).  Each output is one fmaf chain
//     over i ascending from zero -- the CPU oracle's order.
//   - the Hadamard transform needs no shuffles: a thread owns one token (lane) and 16/8/4/2
//     coordinates of one radix group; strides run from D/2 down to 1 in passes of up to 4 bits.
// Weights of 256 output columns (PC/BS blocks) are staged per pass into shared memory as
// Ws[g][i][o] with a 16-byte XOR swizzle, from either global layout ([o][i] or [i][o]).
// No tensor cores: sign bits must reproduce the fp32 fmaf chain.
#include "common.cuh"
#include "hash_common.cuh"

namespace lffn {

// Optional phase clocks (compile with -DLFFN_HB_PHASE_CLOCKS; a profiling build, never the shipped one): thread 0 of
// every CTA adds the clock64 cycles between consecutive marks to a per-phase counter.  Off by default.
#ifdef LFFN_HB_PHASE_CLOCKS
__device__ unsigned long long g_hb_phase[8];
__device__ long long g_hb_last[1024];
__device__ __forceinline__ void hb_mark(int phase) {  // phase < 0: start the clock only
    if (threadIdx.x == 0) {
        const long long now = clock64();
        if (phase >= 0) atomicAdd(&g_hb_phase[phase], (unsigned long long)(now - g_hb_last[blockIdx.x & 1023]));
        g_hb_last[blockIdx.x & 1023] = now;
    }
}
#define HB_MARK(phase) hb_mark(phase)
#else
#define HB_MARK(phase)
#endif
enum { HB_PH_TILE = 0, HB_PH_FMA = 1, HB_PH_HADAMARD = 2, HB_PH_MIX = 3, HB_PH_CODES = 4, HB_PH_CHUNK_WAIT = 5, HB_PH_WRITEBACK = 6 };

constexpr int HB_M = 32;        // tokens per tile
constexpr int HB_MP = 36;       // padded tokens per coordinate row
constexpr int HB_THREADS = 256;
constexpr int HB_CARRY = 16;
constexpr int HB_WFLOATS = 16384;  // staged weights per pass: PC * BS floats
constexpr int HB_LN_FLOATS = 2 * HB_M;  // LayerNorm statistics (mean, 1/sigma) of the tile's tokens

template <int RADIX>
__device__ __forceinline__ void radix_butterflies(float (&v)[RADIX]) {
#ifdef LFFN_HB_SCALAR_BUTTERFLIES
#pragma unroll
    for (int s = RADIX / 2; s >= 1; s >>= 1) {
#pragma unroll
        for (int q = 0; q < RADIX; q++) {
            if ((q & s) == 0) {
                const float a = v[q], b = v[q + s];
                v[q] = __fadd_rn(a, b);
                v[q + s] = __fsub_rn(a, b);
            }
        }
    }
#else
    reg_butterflies<RADIX>(v);  // two butterflies per packed instruction, same roundings
#endif
}

// One pass of the transform over bits [lo, lo+nb) of the coordinate index, RADIX = 2^nb.
// gdst, when given: the transformed tile also goes to global memory as [D][HB_M] (token rows of 128 bytes, written
// straight from the registers that hold the pass's results).
template <int RADIX, int NW>
__device__ __forceinline__ void fwht_pass(float *Y, int D, int lo, float scale, int warp, int lane, float *gdst = nullptr) {
    const int ngroups = D / RADIX;
    const int lo_mask = (1 << lo) - 1;
    for (int gi = warp; gi < ngroups; gi += NW) {
        const int base = ((gi >> lo) * RADIX << lo) | (gi & lo_mask);
        float v[RADIX];
#pragma unroll
        for (int q = 0; q < RADIX; q++) v[q] = Y[(base + (q << lo)) * HB_MP + lane];
        radix_butterflies<RADIX>(v);
        if (scale != 1.f) {
#pragma unroll
            for (int q = 0; q < RADIX; q += 2) mul2(v[q], v[q + 1], v[q], v[q + 1], scale, scale);
        }
#pragma unroll
        for (int q = 0; q < RADIX; q++) Y[(base + (q << lo)) * HB_MP + lane] = v[q];
        if (gdst != nullptr) {
#pragma unroll
            for (int q = 0; q < RADIX; q++) gdst[(size_t)(base + (q << lo)) * HB_M + lane] = v[q];
        }
    }
}

template <int NW = HB_THREADS / 32>
__device__ __forceinline__ void fwht_tile(float *Y, int D, float scale, int warp, int lane, float *gdst = nullptr) {
    int bits = 31 - __clz(D);
    // up to 5 bits (radix 32) per pass, split evenly: 10 bits = 5 + 5, 9 = 5 + 4
    while (bits > 0) {
        const int left = (bits + 4) / 5;
        const int nb = (bits + left - 1) / left;
        const int lo = bits - nb;
        const float sc = lo == 0 ? scale : 1.f;
        float *gd = lo == 0 ? gdst : nullptr;  // the last pass holds the finished values
        if (nb == 5) fwht_pass<32, NW>(Y, D, lo, sc, warp, lane, gd);
        else if (nb == 4) fwht_pass<16, NW>(Y, D, lo, sc, warp, lane, gd);
        else if (nb == 3) fwht_pass<8, NW>(Y, D, lo, sc, warp, lane, gd);
        else if (nb == 2) fwht_pass<4, NW>(Y, D, lo, sc, warp, lane, gd);
        else fwht_pass<2, NW>(Y, D, lo, sc, warp, lane, gd);
        bits = lo;
        __syncthreads();
    }
}

// ---- tile phases shared by the two kernels (THREADS threads, NW = THREADS / 32 warps) ---------------------------------
// Start of a rotation: keep the last coordinates of the previous rotation (for a table that straddles the
// boundary), then load the tile transposed and zero-padded.  The caller synchronises afterwards.
// lnstat [2][HB_M]: mean and 1/sqrt(var + eps) of every token of the tile, filled here when the LayerNorm prologue
// is on (a warp owns a token's row: two passes over it for the statistics, a third writes the normalised values).
template <typename XT, int THREADS>
__device__ __forceinline__ void tile_load(float *dst, const HashArgs &a, long long n0, int mt, int D, float *lnstat) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int mm = warp; mm < HB_M; mm += THREADS / 32) {
        const XT *xrow = static_cast<const XT *>(a.x) + (n0 + mm) * a.d_in;
        if (a.ln_g != nullptr) {
            float mean = 0.f, rstd = 1.f;
            if (mm < mt) {
                float s = 0.f;
                for (int e = lane; e < a.d_in; e += 32) s += Elem<XT>::load1(xrow + e);
                mean = warp_sum(s) / (float)a.d_in;
                float q = 0.f;
                for (int e = lane; e < a.d_in; e += 32) {
                    const float c = Elem<XT>::load1(xrow + e) - mean;
                    q = fmaf(c, c, q);
                }
                rstd = 1.f / sqrtf(warp_sum(q) / (float)a.d_in + a.ln_eps);
            }
            if (lane == 0) {
                lnstat[mm] = mean;
                lnstat[HB_M + mm] = rstd;
            }
            for (int e = lane; e < D; e += 32)
                dst[e * HB_MP + mm] = (mm < mt && e < a.d_in)
                                          ? ln_apply(Elem<XT>::load1(xrow + e), mean, rstd, __ldg(a.ln_g + e),
                                                     a.ln_b != nullptr ? __ldg(a.ln_b + e) : 0.f)
                                          : 0.f;
        } else {
#pragma unroll 8
            for (int e = lane; e < D; e += 32)
                dst[e * HB_MP + mm] = (mm < mt && e < a.d_in) ? Elem<XT>::load1(xrow + e) : 0.f;
        }
    }
}

__device__ __forceinline__ void tile_save_carry(const float *Y, float *carry, int D, int threads) {
    for (int i = threadIdx.x; i < HB_CARRY * HB_M; i += threads) {
        const int e = i / HB_M, mm = i % HB_M;
        carry[e * HB_MP + mm] = Y[(D - HB_CARRY + e) * HB_MP + mm];
    }
}

template <typename XT, int THREADS>
__device__ __forceinline__ void tile_begin_rotation(float *Y, float *carry, const HashArgs &a, long long n0, int mt, int D,
                                                    float *lnstat) {
    __syncthreads();
    tile_save_carry(Y, carry, D, THREADS);
    __syncthreads();
    tile_load<XT, THREADS>(Y, a, n0, mt, D, lnstat);
}

// End of a rotation: z = fl(fl(mix_a * y) + fl(mix_b * u)) + bias in place, then codes and weights of the
// tables that end inside this rotation (lane = token, warps stride over tables).  Xs, when not null, is a copy of
// the input tile in the layout of Y: u comes from there instead of global memory, and when no table straddles a
// rotation boundary and z itself is not wanted the mix is folded into the code/weight step (Y is not rewritten).
template <typename XT, int THREADS>
__device__ __forceinline__ void tile_end_rotation(float *Y, const float *carry, const HashArgs &a, long long n0, int mt,
                                                  int D, int r, const float *lnstat, const float *Xs = nullptr) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int k = a.k;
    const int m = a.weight_mode == LFFN_WEIGHT_SOFT_FLIP ? k + 1 : 1;
    const long long g_lo = (long long)a.t_begin * k, g_hi = (long long)(a.t_begin + a.t_count) * k;
    const long long out_pitch = (long long)a.t_count * m;
    const long long c_lo = (long long)r * D, c_hi = c_lo + D;
    const bool fused = Xs != nullptr && a.z_out == nullptr && D % k == 0;
    if (Xs != nullptr && !fused) {
        for (int e = warp; e < D; e += THREADS / 32) {  // lane = token
            const long long g = c_lo + e;
            float z = __fadd_rn(__fmul_rn(a.mix_a, Y[e * HB_MP + lane]), __fmul_rn(a.mix_b, Xs[e * HB_MP + lane]));
            if (a.bias != nullptr && g < (long long)a.T * k) z = __fadd_rn(z, __ldg(a.bias + g));
            Y[e * HB_MP + lane] = z;
        }
        __syncthreads();
        if (a.z_out != nullptr) {  // rows of z with the lanes over coordinates: 128-byte stores
            for (int mm = warp; mm < mt; mm += THREADS / 32) {
                float *zrow = a.z_out + (n0 + mm) * (g_hi - g_lo);
                for (int e = lane; e < D; e += 32) {
                    const long long g = c_lo + e;
                    if (g >= g_lo && g < g_hi) zrow[g - g_lo] = Y[e * HB_MP + mm];
                }
            }
        }
    } else if (!fused) {
        for (int mm = warp; mm < HB_M; mm += THREADS / 32) {
            const XT *xrow = static_cast<const XT *>(a.x) + (n0 + mm) * a.d_in;
            for (int e = lane; e < D; e += 32) {
                float u = (mm < mt && e < a.d_in) ? Elem<XT>::load1(xrow + e) : 0.f;
                if (a.ln_g != nullptr && mm < mt && e < a.d_in)  // the statistics of tile_load
                    u = ln_apply(u, lnstat[mm], lnstat[HB_M + mm], __ldg(a.ln_g + e), a.ln_b != nullptr ? __ldg(a.ln_b + e) : 0.f);
                const long long g = c_lo + e;
                float z = __fadd_rn(__fmul_rn(a.mix_a, Y[e * HB_MP + mm]), __fmul_rn(a.mix_b, u));
                if (a.bias != nullptr && g < (long long)a.T * k) z = __fadd_rn(z, __ldg(a.bias + g));
                Y[e * HB_MP + mm] = z;
                if (a.z_out != nullptr && mm < mt && g >= g_lo && g < g_hi)
                    a.z_out[(n0 + mm) * (g_hi - g_lo) + (g - g_lo)] = z;
            }
        }
        __syncthreads();
    }
    HB_MARK(HB_PH_MIX);
    long long t_first = c_lo / k;
    if (t_first < a.t_begin) t_first = a.t_begin;
    long long t_end = c_hi / k;
    if (t_end > a.t_begin + a.t_count) t_end = a.t_begin + a.t_count;
    if (lane < mt && a.idx_out != nullptr) {
        auto emit = [&](long long t, int wm, int32_t *io, float *wo) {
            const int local0 = (int)(t * k - c_lo);
            auto get = [&](int j) -> float {
                const int e = local0 + j;
                if (fused) {  // no straddling table here: e >= 0
                    float z = __fadd_rn(__fmul_rn(a.mix_a, Y[e * HB_MP + lane]), __fmul_rn(a.mix_b, Xs[e * HB_MP + lane]));
                    if (a.bias != nullptr) z = __fadd_rn(z, __ldg(a.bias + c_lo + e));
                    return z;
                }
                return e >= 0 ? Y[e * HB_MP + lane] : carry[(HB_CARRY + e) * HB_MP + lane];
            };
            emit_table(get, k, a.bit_order, wm, a.tau, (int32_t)((t - a.t_begin) << k), false, 0, io, wo);
        };
        // the common case (8-bit codes, mix folded in, input tile in shared memory): the table's coordinates go to
        // registers two at a time with packed multiplies and adds, same roundings as `get` above
        auto emit8 = [&](long long t, int wm, int32_t *io, float *wo) {
            const int local0 = (int)(t * 8 - c_lo);
            float z[8];
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                const int e = local0 + j;
                // scalar multiplies: a packed product feeding a packed add would be contracted (see mul2)
                const float p0 = __fmul_rn(a.mix_a, Y[e * HB_MP + lane]), p1 = __fmul_rn(a.mix_a, Y[(e + 1) * HB_MP + lane]);
                const float q0 = __fmul_rn(a.mix_b, Xs[e * HB_MP + lane]), q1 = __fmul_rn(a.mix_b, Xs[(e + 1) * HB_MP + lane]);
                add2(z[j], z[j + 1], p0, p1, q0, q1);
                if (a.bias != nullptr) add2(z[j], z[j + 1], z[j], z[j + 1], __ldg(a.bias + c_lo + e), __ldg(a.bias + c_lo + e + 1));
            }
            emit_table_k<8>(z, a.bit_order, wm, a.tau, (int32_t)((t - a.t_begin) << 8), io, wo);
        };
        const bool vec4 = m == 1 && (out_pitch & 3) == 0 && ((reinterpret_cast<uintptr_t>(a.idx_out) & 15u) == 0) &&
                          ((reinterpret_cast<uintptr_t>(a.w_out) & 15u) == 0);
        if (vec4 && fused && k == 8 && Xs != nullptr) {
            const int wm = a.weight_mode == LFFN_WEIGHT_ONES ? LFFN_WEIGHT_ONES : LFFN_WEIGHT_SCORE;
            const long long q_first = (t_first - a.t_begin) >> 2, q_end = (t_end - a.t_begin + 3) >> 2;
            for (long long q = q_first + warp; q < q_end; q += THREADS / 32) {
                const long long tb = a.t_begin + q * 4;
                const long long o = (n0 + lane) * out_pitch + q * 4;
                if (tb >= t_first && tb + 4 <= t_end) {
                    int32_t ci[4];
                    float cw[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) emit8(tb + u, wm, ci + u, cw + u);
                    *reinterpret_cast<int4 *>(a.idx_out + o) = make_int4(ci[0], ci[1], ci[2], ci[3]);
                    *reinterpret_cast<float4 *>(a.w_out + o) = make_float4(cw[0], cw[1], cw[2], cw[3]);
                } else {
                    for (int u = 0; u < 4; u++)
                        if (tb + u >= t_first && tb + u < t_end) emit8(tb + u, wm, a.idx_out + o + u, a.w_out + o + u);
                }
            }
        } else if (vec4) {
            // m == 1 rules out the soft-flip mode: naming the two remaining modes lets the compiler drop that branch
            const int wm = a.weight_mode == LFFN_WEIGHT_ONES ? LFFN_WEIGHT_ONES : LFFN_WEIGHT_SCORE;
            // a warp takes four consecutive tables at a time and each lane (token) writes their codes and weights
            // with one 16-byte store each
            const long long q_first = (t_first - a.t_begin) >> 2, q_end = (t_end - a.t_begin + 3) >> 2;
            for (long long q = q_first + warp; q < q_end; q += THREADS / 32) {
                const long long tb = a.t_begin + q * 4;
                const long long o = (n0 + lane) * out_pitch + q * 4;
                if (tb >= t_first && tb + 4 <= t_end) {
                    int32_t ci[4];
                    float cw[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) emit(tb + u, wm, ci + u, cw + u);
                    *reinterpret_cast<int4 *>(a.idx_out + o) = make_int4(ci[0], ci[1], ci[2], ci[3]);
                    *reinterpret_cast<float4 *>(a.w_out + o) = make_float4(cw[0], cw[1], cw[2], cw[3]);
                } else {
                    for (int u = 0; u < 4; u++)
                        if (tb + u >= t_first && tb + u < t_end) emit(tb + u, wm, a.idx_out + o + u, a.w_out + o + u);
                }
            }
        } else {
            for (long long t = t_first + warp; t < t_end; t += THREADS / 32) {
                const long long o = (n0 + lane) * out_pitch + (t - a.t_begin) * m;
                emit(t, a.weight_mode, a.idx_out + o, a.w_out + o);
            }
        }
    }
}

template <typename XT>
__global__ void __launch_bounds__(HB_THREADS, 1) hash_block_kernel(HashArgs a, int BS, int transpose_w) {
    extern __shared__ __align__(16) float smem[];
    const int D = a.D;
    float *Y = smem;                         // [D][HB_MP]
    float *Ws = Y + (size_t)D * HB_MP;       // [PC/BS][BS][BS] swizzled
    float *carry = Ws + HB_WFLOATS;          // [HB_CARRY][HB_MP]
    float *lnstat = carry + HB_CARRY * HB_MP;  // [2][HB_M]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int PC = min(D, BS <= 64 ? 256 : HB_WFLOATS / BS);  // columns per pass
    const int bs4mask = BS / 4 - 1;
    const long long ntiles = (a.N + HB_M - 1) / HB_M;

    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const long long n0 = tile * HB_M;
        const int mt = (int)min((long long)HB_M, a.N - n0);  // valid tokens in the tile
        for (int r = a.r_lo; r <= a.r_hi; r++) {
            tile_begin_rotation<XT, HB_THREADS>(Y, carry, a, n0, mt, D, lnstat);
            __syncthreads();
            for (int s = 0; s < a.S; s++) {
                const float *wstage = a.w + ((long long)r * a.S + s) * D * BS;
                for (int col0 = 0; col0 < D; col0 += PC) {
                    // stage PC/BS weight blocks as Ws[g][i][o], 16-byte XOR swizzle on o
                    const float *wsrc = wstage + (long long)col0 * BS;
                    for (int L = tid; L < PC * BS; L += HB_THREADS) {
                        const int g = L / (BS * BS), rem = L % (BS * BS);
                        const int p = rem / BS, q = rem % BS;
                        const int i = transpose_w ? p : q, o = transpose_w ? q : p;
                        Ws[g * BS * BS + i * BS + ((((o >> 2) ^ (i & bs4mask)) << 2) | (o & 3))] = __ldg(wsrc + L);
                    }
                    __syncthreads();
                    // PC output columns x 32 tokens = PC items of 8 tokens x 4 columns: at most one per thread
                    const bool active = tid < PC;
                    const int cq = tid % (PC / 4), tq = tid / (PC / 4);
                    const int c = cq * 4, g = c / BS, o4 = (c % BS) >> 2;
                    float acc[8][4];
#pragma unroll
                    for (int p = 0; p < 8; p++)
#pragma unroll
                        for (int q = 0; q < 4; q++) acc[p][q] = 0.f;
                    if (active) {
                        const float *yb = Y + (size_t)(col0 + g * BS) * HB_MP + tq * 8;
                        const float *wb = Ws + g * BS * BS;
#pragma unroll 4
                        for (int i = 0; i < BS; i++) {
                            const float4 x0 = *reinterpret_cast<const float4 *>(yb + i * HB_MP);
                            const float4 x1 = *reinterpret_cast<const float4 *>(yb + i * HB_MP + 4);
                            const float4 w4 = *reinterpret_cast<const float4 *>(wb + i * BS + ((o4 ^ (i & bs4mask)) << 2));
                            const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
                            const float wv[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                            for (int p = 0; p < 8; p++)
#pragma unroll
                                for (int q = 0; q < 4; q++) acc[p][q] = fmaf(xs[p], wv[q], acc[p][q]);
                        }
                    }
                    __syncthreads();  // all reads of this pass's input columns are done before they are overwritten
                    if (active) {
                        float *yo = Y + (size_t)(col0 + c) * HB_MP + tq * 8;
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            *reinterpret_cast<float4 *>(yo + q * HB_MP) = make_float4(acc[0][q], acc[1][q], acc[2][q], acc[3][q]);
                            *reinterpret_cast<float4 *>(yo + q * HB_MP + 4) = make_float4(acc[4][q], acc[5][q], acc[6][q], acc[7][q]);
                        }
                    }
                    __syncthreads();
                }
                fwht_tile(Y, D, a.had_scale, warp, lane);
            }
            tile_end_rotation<XT, HB_THREADS>(Y, carry, a, n0, mt, D, r, lnstat);
        }
    }
}

// ---- fast path: 64 x 64 blocks, weights stored [block][i][o] ------------------------------------------
// Same tile layout and arithmetic as hash_block_kernel; what changes is how the weights travel and how the
// multiply-adds are issued.  Weights stream through two 32 KB shared buffers in chunks of (NBLK blocks) x (CR
// input rows) x (64 outputs).  A chunk is NBLK contiguous pieces of global memory, so one thread fetches it with
// NBLK bulk copies (cp.async.bulk, the TMA unit) that signal a "full" mbarrier by byte count; every warp reports on
// an "empty" mbarrier when it has finished with a chunk, and the next fetch into that buffer waits for the 16
// reports.  The fetch runs one chunk ahead of the arithmetic across passes, stages and rotations, so the Hadamard
// passes hide the next stage's first chunk, and there is no CTA-wide barrier inside the multiply-add loop: the
// columns a warp overwrites after a pass are read only by that same warp (two blocks x one token octet).
// The 8 x 4 register tile is held as 16 packed pairs and updated with fma.rn.f32x2 (two IEEE fp32 fused
// multiply-adds per instruction).  Each output is still one fmaf chain over i ascending.
//
// Every mbarrier wait is a bounded poll: when the bound is hit the thread sets LFFN_STATUS_TIMEOUT in the device
// status word and leaves the kernel (the outputs of that launch are then incomplete).
__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
constexpr int MBAR_POLL_LIMIT = 1 << 22;  // polls of a few tens of ns each: gives up after about 0.1 - 0.2 s
__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, unsigned parity, int limit = MBAR_POLL_LIMIT) {
    const unsigned addr = smem_u32(bar);
    for (int it = 0; it < limit; it++) {
        unsigned done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
// global -> shared bulk copy (16-byte aligned addresses, size a multiple of 16) that adds its byte count to `bar`
__device__ __forceinline__ void bulk_copy_g2s(void *smem_dst, const void *gmem_src, unsigned bytes, unsigned long long *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(__cvta_generic_to_global(gmem_src)), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// 4-byte asynchronous copy global -> shared (zero fill when !valid: nothing is read from gsrc then)
__device__ __forceinline__ void cp_async4(float *smem_dst, const float *gsrc, bool valid) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_u32(smem_dst)), "l"(__cvta_generic_to_global(gsrc)),
                 "r"(valid ? 4u : 0u)
                 : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ unsigned long long dup2(float w) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %1};" : "=l"(r) : "f"(w));
    return r;
}
__device__ __forceinline__ void ffma2(unsigned long long &acc, unsigned long long a, unsigned long long b) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}

constexpr int HF_CHUNK_FLOATS = 4 * 32 * 64;  // 4 blocks x 32 rows x 64 outputs
#ifndef LFFN_HB_NBUF
#define LFFN_HB_NBUF 2
#endif
constexpr int HF_NBUF = LFFN_HB_NBUF;          // weight buffers in the ring (2 or 4), 64 KB together
constexpr int HF_BAR_FLOATS = 4 * HF_NBUF;     // a full and an empty mbarrier per buffer, behind the carry rows

// THREADS = columns per pass (one 8 x 4 item per thread): 256 threads work on 4 blocks x 32-row chunks, 512 threads
// on 8 blocks x 16-row chunks; the chunk is 32 KB either way.
// X0: shared memory has room for a second [D][HB_MP] array (D <= 512): the input tile is loaded once per tile and
// kept there; the first stage of every rotation reads it directly and the mix at the end of a rotation takes u
// from it, instead of eight passes over the tile's rows in global memory per tile.  In mode 2 the second array is the
// other half of a double buffer: the gradient tile of the next unit is fetched into it with asynchronous copies
// while the current unit is being worked on.
//
// MODE selects what the tile pipeline is used for:
//   0  the hashing stage itself (codes, weights, optionally z)
//   1  the same forward walk for training: the input y_s of every stage s of rotation r is saved to
//      a.act_out[r - r_lo][s][tile] ([D][32] per tile, the shared-memory layout without its padding); z too when
//      a.z_out is given, no codes
//   2  the backward walk of one rotation: g = mix_a * dz, then for s = S-1 .. 0: g <- H g * had_scale, saved to
//      a.act_out[s][tile] (this is the gradient at the output of stage s's multiply), g <- g W[r, s] (a.w is then
//      the parameter in its own [o][i] order, which is input-major for this product); the result, the gradient
//      with respect to the rotation's input, goes to a.du_out[tile]
// Mode 2 is launched for one rotation at a time (r_lo == r_hi).  In modes 1 and 2 the tiles of the later stages are
// written out by the last pass of the transform that produces them (fwht_pass, gdst).
template <int THREADS>
__device__ __forceinline__ void tile_save(const float *Y, float *dst, int D) {
    for (int i = threadIdx.x; i < D * HB_M; i += THREADS) dst[i] = Y[(i >> 5) * HB_MP + (i & 31)];
}

template <typename XT, int THREADS, bool X0, int MODE = 0>
__global__ void __launch_bounds__(THREADS, 1) hash_block64_kernel(HashArgs a) {
    constexpr int PC = THREADS;            // columns per pass
    constexpr int CHUNK = 2 * HF_CHUNK_FLOATS / HF_NBUF;  // floats per weight buffer
    constexpr int CR = CHUNK / PC;         // input rows per chunk
    constexpr int NBLK = PC / 64;          // blocks per pass
    constexpr int NW = THREADS / 32;
    extern __shared__ __align__(16) float smem[];
    const int D = a.D;
    float *Y = smem;                              // [D][HB_MP]
    float *Wb = Y + (size_t)D * HB_MP;            // 2 x HF_CHUNK_FLOATS
    float *carry = Wb + 2 * HF_CHUNK_FLOATS;      // [HB_CARRY][HB_MP]
    unsigned long long *bars = reinterpret_cast<unsigned long long *>(carry + HB_CARRY * HB_MP);
    unsigned long long *full = bars, *empty = bars + HF_NBUF;  // one pair per weight buffer
    float *lnstat = carry + HB_CARRY * HB_MP + HF_BAR_FLOATS;                // [2][HB_M]
    float *Xs = X0 ? lnstat + HB_LN_FLOATS : nullptr;                         // [D][HB_MP]; mode 2: the other tile buffer
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int NB = D / 64;
    const int cps = (D / PC) * (64 / CR);            // chunks per stage: passes x row slices
    const int nrot = a.r_hi - a.r_lo + 1;
    const long long ntiles = (a.N + HB_M - 1) / HB_M;
    // Work units are (tile, rotation) pairs, tile-major, cut into gridDim.x contiguous ranges of nearly equal length:
    // rotations are independent, so with 512 tiles x 4 rotations on 148 CTAs every CTA gets 13 or 14 units instead of
    // 3 or 4 whole tiles.  When a table can straddle two rotations (k does not divide D) a range holds whole tiles.
    const long long per = (D % a.k == 0) ? 1 : nrot;
    const long long groups = ntiles * nrot / per;
    const long long u_begin = groups * blockIdx.x / gridDim.x * per, u_end = groups * (blockIdx.x + 1) / gridDim.x * per;
    const long long total_chunks = (u_end - u_begin) * a.S * cps;

    if (tid == 0) {
#pragma unroll
        for (int b = 0; b < HF_NBUF; b++) {
            mbar_init(&full[b], 1);
            mbar_init(&empty[b], NW);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // Chunks are consumed in the order (tile, rotation, stage, pass, row slice); the weights do not depend on the
    // tile.  Every thread advances the position of the next chunk (incrementally, no divisions in the loop); chunk c
    // is fetched by lane 0 of warp c % NW, so the wait for the buffer to be free -- for the slowest warp to finish
    // chunk c - HF_NBUF -- falls on a different warp each time instead of making one warp the straggler.
    // Chunk c lives in buffer c % HF_NBUF and is the (c / HF_NBUF)-th use of that buffer's barriers; the fetch
    // runs HF_NBUF - 1 chunks ahead of the arithmetic.
    int nx_r = a.r_lo + (int)(u_begin % nrot), nx_s = 0, nx_p = 0, nx_h = 0;
    auto next_chunk_src = [&]() -> const float * {
        const int s_eff = MODE == 2 ? a.S - 1 - nx_s : nx_s;  // the backward walk takes the stages in reverse
        const float *src = a.w + (((long long)nx_r * a.S + s_eff) * NB + NBLK * nx_p) * 4096 + nx_h * CR * 64;
        if (++nx_h == 64 / CR) {
            nx_h = 0;
            if (++nx_p == D / PC) {
                nx_p = 0;
                if (++nx_s == a.S) {
                    nx_s = 0;
                    if (++nx_r > a.r_hi) nx_r = a.r_lo;
                }
            }
        }
        return src;
    };
    auto fetch_chunk = [&](long long c, const float *src) -> bool {  // one thread
        const int b = (int)(c % HF_NBUF);
        // the buffer's previous chunk, c - HF_NBUF, must have been reported finished by every warp
        if (c >= HF_NBUF && !mbar_wait(&empty[b], (unsigned)(((c - HF_NBUF) / HF_NBUF) & 1))) return false;
        float *dst = Wb + b * CHUNK;
        mbar_arrive_expect_tx(&full[b], CHUNK * sizeof(float));
#pragma unroll
        for (int g = 0; g < NBLK; g++) bulk_copy_g2s(dst + g * (CR * 64), src + (long long)g * 4096, CR * 64 * sizeof(float), &full[b]);
        return true;
    };
    // all threads call this once per chunk, in chunk order; false = the fetching warp timed out and must leave
    auto issue_chunk = [&](long long c) -> bool {
        if (c >= total_chunks) return true;
        const float *src = next_chunk_src();
        if (warp != (int)(c % NW)) return true;
        int ok = 1;
        if (lane == 0) ok = fetch_chunk(c, src) ? 1 : 0;
        return __shfl_sync(FULL, ok, 0) != 0;
    };
    // A thread that gives up first waits (bounded again) for the chunks [from, to) that have been requested but not
    // consumed, so that it does not leave while a bulk copy it issued is still writing into this CTA's shared
    // memory: shared memory is released only when the last thread has left, and every issuer waits for its own copy
    // either in the normal flow or here.
    auto give_up = [&](long long from, long long to) {
        if (a.status != nullptr) atomicOr(a.status, LFFN_STATUS_TIMEOUT);
        cp_async_wait_all();  // this thread's share of a prefetched tile (mode 2), if any
        for (long long c = from; c < to && c < total_chunks; c++)
            mbar_wait(&full[c % HF_NBUF], (unsigned)((c / HF_NBUF) & 1));
    };

    // mode 2 with a second tile buffer: asynchronous, transposing fetch of the gradient tile of (tile_, r_)
    auto request_dz_tile = [&](float *dst, long long tile_, int r_) {
        const long long n0_ = tile_ * HB_M;
        const int mt_ = (int)min((long long)HB_M, a.N - n0_);
        const int dshift = 31 - __clz(D);
        for (int i = tid; i < D * HB_M; i += THREADS) {
            const int e = i & (D - 1), mm = i >> dshift;
            const bool in = mm < mt_ && (long long)r_ * D + e < a.dz_cols;
            cp_async4(dst + e * HB_MP + mm, in ? a.dz + (n0_ + mm) * a.dz_cols + (long long)r_ * D + e : a.dz, in);
        }
    };
    if constexpr (MODE == 2 && X0) {
        if (u_begin < u_end) request_dz_tile(Xs, u_begin / nrot, a.r_lo + (int)(u_begin % nrot));
    }

    long long gc = 0;
    HB_MARK(-1);
#pragma unroll
    for (int c = 0; c < HF_NBUF - 1; c++) issue_chunk(c);  // the first use of a buffer waits for nothing
    long long tile = u_begin / nrot;
    int r = a.r_lo + (int)(u_begin % nrot);
    for (long long u = u_begin; u < u_end; u++) {
        const long long n0 = tile * HB_M;
        const int mt = (int)min((long long)HB_M, a.N - n0);
        const bool first_of_tile = u == u_begin || r == a.r_lo;
        if constexpr (MODE == 2) {
            if constexpr (X0) {
                // The gradient tile of this unit was requested during the previous one (asynchronous 4-byte copies into
                // the second tile buffer, already transposed): wait for it, make that buffer the working tile, and
                // request the next unit's tile into the buffer the previous unit has just finished with.  Read straight
                // from global memory these 64 KB cost a quarter of the kernel in exposed latency.
                cp_async_wait_all();
                __syncthreads();  // every thread's copies have landed; the previous unit has finished with Y
                float *t = Y;
                Y = Xs;
                Xs = t;
                if (u + 1 < u_end) {
                    const int rn = r + 1 > a.r_hi ? a.r_lo : r + 1;
                    request_dz_tile(Xs, rn == a.r_lo ? tile + 1 : tile, rn);
                }
                if (a.mix_a != 1.f) {
                    for (int i = tid; i < D * HB_M; i += THREADS) {
                        float *p = Y + (i >> 5) * HB_MP + (i & 31);
                        *p = __fmul_rn(a.mix_a, *p);
                    }
                }
            } else {
                __syncthreads();  // the previous unit has finished with Y
                const int dshift = 31 - __clz(D);
#pragma unroll 8
                for (int i = tid; i < D * HB_M; i += THREADS) {
                    const int e = i & (D - 1), mm = i >> dshift;
                    const bool in = mm < mt && (long long)r * D + e < a.dz_cols;
                    const float gv = in ? __ldg(a.dz + (n0 + mm) * a.dz_cols + (long long)r * D + e) : 0.f;
                    Y[e * HB_MP + mm] = in ? __fmul_rn(a.mix_a, gv) : 0.f;
                }
            }
        } else if constexpr (X0) {
            if (first_of_tile) {
                __syncthreads();  // the previous unit has finished reading Xs
                tile_load<XT, THREADS>(Xs, a, n0, mt, D, lnstat);
            } else if (D % a.k != 0) {
                __syncthreads();
                tile_save_carry(Y, carry, D, THREADS);
            }
        } else {
            tile_begin_rotation<XT, THREADS>(Y, carry, a, n0, mt, D, lnstat);
        }
        __syncthreads();  // the tile (and the carry rows) are in place
        HB_MARK(HB_PH_TILE);
        // one stage's block-diagonal multiply: Y <- blockdiag(W) ysrc, pass by pass; false = a bounded wait ran out
        auto multiply_stage = [&](const float *ysrc) -> bool {
            const int cq = tid % (PC / 4), tq = tid / (PC / 4);   // PC/4 column quads x 4 token octets
            const int g = cq >> 4, o4 = cq & 15;
            for (int p = 0; p < D / PC; p++) {
                const int col0 = p * PC;
                unsigned long long acc[4][4];               // [token pair][column]
#pragma unroll
                for (int pp = 0; pp < 4; pp++)
#pragma unroll
                    for (int q = 0; q < 4; q++) acc[pp][q] = 0ull;
                for (int h = 0; h < 64 / CR; h++) {
                    HB_MARK(HB_PH_FMA);
                    if (!issue_chunk(gc + HF_NBUF - 1)) {  // that chunk was not requested; the ones before it were
                        give_up(gc, gc + HF_NBUF - 1);
                        return false;
                    }
                    const int buf = (int)(gc % HF_NBUF);
                    if (!mbar_wait(&full[buf], (unsigned)((gc / HF_NBUF) & 1))) {  // chunk gc has landed
                        give_up(gc, gc + HF_NBUF);
                        return false;
                    }
                    HB_MARK(HB_PH_CHUNK_WAIT);
                    const float *wb = Wb + buf * CHUNK + g * (CR * 64);
                    const float *yb = ysrc + (size_t)(col0 + g * 64 + h * CR) * HB_MP + tq * 8;
#pragma unroll 16
                    for (int il = 0; il < CR; il++) {
                        const ulonglong2 x0 = *reinterpret_cast<const ulonglong2 *>(yb + il * HB_MP);
                        const ulonglong2 x1 = *reinterpret_cast<const ulonglong2 *>(yb + il * HB_MP + 4);
                        const float4 w4 = *reinterpret_cast<const float4 *>(wb + il * 64 + (o4 << 2));
                        const unsigned long long wq[4] = {dup2(w4.x), dup2(w4.y), dup2(w4.z), dup2(w4.w)};
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            ffma2(acc[0][q], x0.x, wq[q]);
                            ffma2(acc[1][q], x0.y, wq[q]);
                            ffma2(acc[2][q], x1.x, wq[q]);
                            ffma2(acc[3][q], x1.y, wq[q]);
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty[buf]);  // this warp is done with the buffer
                    gc++;
                }
                HB_MARK(HB_PH_FMA);
                // the 64 input columns of a block x 8 tokens are read by one half-warp, the one that overwrites them
                __syncwarp();
                float *yo = Y + (size_t)(col0 + cq * 4) * HB_MP + tq * 8;
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    *reinterpret_cast<ulonglong2 *>(yo + q * HB_MP) = make_ulonglong2(acc[0][q], acc[1][q]);
                    *reinterpret_cast<ulonglong2 *>(yo + q * HB_MP + 4) = make_ulonglong2(acc[2][q], acc[3][q]);
                }
            }
            return true;
        };
        const size_t tile_floats = (size_t)D * HB_M;
        if constexpr (MODE == 2) {
            for (int sb = 0; sb < a.S; sb++) {
                const int s = a.S - 1 - sb;
                // the transformed gradient is saved by the transform's last pass itself (ends with a CTA barrier)
                fwht_tile<NW>(Y, D, a.had_scale, warp, lane,
                              a.act_out + ((size_t)((r - a.r_lo) * a.S + s) * ntiles + tile) * tile_floats);
                HB_MARK(HB_PH_HADAMARD);
                if (!multiply_stage(Y)) return;
                __syncthreads();
                HB_MARK(HB_PH_WRITEBACK);
            }
            tile_save<THREADS>(Y, a.du_out + (size_t)tile * tile_floats, D);
        } else {
            for (int s = 0; s < a.S; s++) {
                const float *ysrc = (X0 && s == 0) ? Xs : Y;
                if constexpr (MODE == 1) {
                    // the input of stage 0 is saved here; the inputs of the later stages by the transform before them
                    if (s == 0) {
                        tile_save<THREADS>(ysrc, a.act_out + ((size_t)(r - a.r_lo) * a.S * ntiles + tile) * tile_floats, D);
                        if (!X0) __syncthreads();  // ysrc is Y: read before the multiply's write-back overwrites it
                    }
                }
                if (!multiply_stage(ysrc)) return;
                __syncthreads();
                HB_MARK(HB_PH_WRITEBACK);
                fwht_tile<NW>(Y, D, a.had_scale, warp, lane,
                              (MODE == 1 && s + 1 < a.S)
                                  ? a.act_out + ((size_t)((r - a.r_lo) * a.S + s + 1) * ntiles + tile) * tile_floats
                                  : nullptr);
                HB_MARK(HB_PH_HADAMARD);
            }
            // mode 1 may be asked for z as well (training's forward pass keeps the stage inputs for its backward)
            if (MODE == 0 || a.z_out != nullptr) tile_end_rotation<XT, THREADS>(Y, carry, a, n0, mt, D, r, lnstat, Xs);
        }
#ifdef LFFN_HB_PHASE_CLOCKS
        __syncthreads();
#endif
        HB_MARK(HB_PH_CODES);
        if (++r > a.r_hi) {
            r = a.r_lo;
            tile++;
        }
    }
}

// Self-test of the bounded wait: one thread waits on an mbarrier that nobody will ever arrive on (no copy is in
// flight, nothing else runs), with a small poll limit.  The wait must run out, set LFFN_STATUS_TIMEOUT and return,
// leaving the context usable.
__global__ void bounded_wait_selftest_kernel(int poll_limit, uint32_t *status) {
    __shared__ unsigned long long bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (!mbar_wait(&bar, 0u, poll_limit)) atomicOr(status, LFFN_STATUS_TIMEOUT);
    }
}

int launch_bounded_wait_selftest(int poll_limit, cudaStream_t st) {
    uint32_t *status = status_word();
    LFFN_REQUIRE(status != nullptr, LFFN_ERR_CUDA, "cannot locate the device status word");
    bounded_wait_selftest_kernel<<<1, 32, 0, st>>>(poll_limit, status);
    LFFN_CHECK_CUDA(cudaGetLastError());
    return LFFN_OK;
}

// The tile pipeline in its training modes (see hash_block64_kernel): mode 1 saves every stage's input, mode 2 walks
// one rotation backwards.  64 x 64 blocks, D a multiple of 256, a.w input-major for the product at hand.
int launch_hash_block64_mode(const HashArgs &a, int mode, int x_dtype, cudaStream_t st) {
    LFFN_REQUIRE(a.D % 256 == 0 && a.D >= 256 && a.D <= 1024 && (reinterpret_cast<uintptr_t>(a.w) & 15u) == 0,
                 LFFN_ERR_UNSUPPORTED, "block-diagonal backward: D = %d must be 256, 512 or 1024 and the weights 16-byte aligned", a.D);
    LFFN_REQUIRE((mode == 1 || (mode == 2 && a.r_lo == a.r_hi)) && a.k == 1, LFFN_ERR_INVALID_ARG,
                 "block-diagonal backward: mode 1, or mode 2 with one rotation per launch; k = 1");
    const long long ntiles = (a.N + HB_M - 1) / HB_M;
    const long long groups = ntiles * (a.r_hi - a.r_lo + 1);  // (tile, rotation) work units
    long long grid = num_sms();
    if (grid > groups) grid = groups;
    if (grid < 1) grid = 1;
    const bool wide = a.D % 512 == 0;
    const size_t smem_b = ((size_t)a.D * HB_MP + HB_WFLOATS + HB_CARRY * HB_MP + HB_LN_FLOATS + HF_BAR_FLOATS) * sizeof(float);
    const size_t smem_x0 = smem_b + (size_t)a.D * HB_MP * sizeof(float);
    const bool x0 = smem_x0 <= 227 * 1024;  // room for a second tile: the resident input (mode 1), the prefetched gradient tile (mode 2)
    const size_t smem_k = x0 ? smem_x0 : smem_b;
    void (*kern)(HashArgs) = nullptr;
    if (mode == 2) {
        kern = wide ? (x0 ? hash_block64_kernel<float, 512, true, 2> : hash_block64_kernel<float, 512, false, 2>)
                    : (x0 ? hash_block64_kernel<float, 256, true, 2> : hash_block64_kernel<float, 256, false, 2>);
    } else if (x_dtype == LFFN_F32) {
        kern = wide ? (x0 ? hash_block64_kernel<float, 512, true, 1> : hash_block64_kernel<float, 512, false, 1>)
                    : (x0 ? hash_block64_kernel<float, 256, true, 1> : hash_block64_kernel<float, 256, false, 1>);
    } else if (x_dtype == LFFN_BF16) {
        kern = wide ? (x0 ? hash_block64_kernel<__nv_bfloat16, 512, true, 1> : hash_block64_kernel<__nv_bfloat16, 512, false, 1>)
                    : (x0 ? hash_block64_kernel<__nv_bfloat16, 256, true, 1> : hash_block64_kernel<__nv_bfloat16, 256, false, 1>);
    } else {
        set_error("block-diagonal backward: unknown x dtype %d", x_dtype);
        return LFFN_ERR_INVALID_ARG;
    }
    LFFN_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_k));
    kern<<<(unsigned)grid, wide ? 512 : 256, smem_k, st>>>(a);
    LFFN_CHECK_CUDA(cudaGetLastError());
    return LFFN_OK;
}

int launch_hash_block(const HashArgs &a, int BS, int transpose_w, int x_dtype, cudaStream_t st) {
    if (BS < 4 || BS > 128 || (BS & (BS - 1)) != 0 || a.D % BS != 0) {
        set_error("hash_fwd: block size %d unsupported (1, or a power of two in [4, 128] dividing D)", BS);
        return LFFN_ERR_UNSUPPORTED;
    }
    if (a.D < 64 || a.D > 1024 || (a.D & (a.D - 1)) != 0) {
        set_error("hash_fwd: block-diagonal projection supports D a power of two in [64, 1024], got %d", a.D);
        return LFFN_ERR_UNSUPPORTED;
    }
    const size_t smem = ((size_t)a.D * HB_MP + HB_WFLOATS + HB_CARRY * HB_MP + HB_LN_FLOATS) * sizeof(float);
    const long long ntiles = (a.N + HB_M - 1) / HB_M;
    long long grid = num_sms();
    if (grid > ntiles) grid = ntiles;
    if (grid < 1) grid = 1;
    if (BS == 64 && transpose_w && a.D % 256 == 0 && (reinterpret_cast<uintptr_t>(a.w) & 15u) == 0) {
        static_assert(2 * HF_CHUNK_FLOATS == HB_WFLOATS, "same shared-memory footprint as the generic kernel");
        const bool wide = a.D % 512 == 0;   // 512 threads: 16 warps per SM instead of 8
        // the kernel splits (tile, rotation) units, or whole tiles when k does not divide D, evenly over the grid
        const long long nrot = a.r_hi - a.r_lo + 1;
        const long long groups = a.D % a.k == 0 ? ntiles * nrot : ntiles;
        grid = num_sms();
        if (grid > groups) grid = groups;
        if (grid < 1) grid = 1;
        const int threads = wide ? 512 : 256;
        const size_t smem_b = smem + HF_BAR_FLOATS * sizeof(float);              // + the mbarriers (the statistics sit behind them)
        const size_t smem_x0 = smem_b + (size_t)a.D * HB_MP * sizeof(float);  // + the resident copy of the input tile
        const bool x0 = smem_x0 <= 227 * 1024;
        const size_t smem_k = x0 ? smem_x0 : smem_b;
        void (*kern)(HashArgs) = nullptr;
        if (x_dtype == LFFN_F32) {
            kern = wide ? (x0 ? hash_block64_kernel<float, 512, true> : hash_block64_kernel<float, 512, false>)
                        : (x0 ? hash_block64_kernel<float, 256, true> : hash_block64_kernel<float, 256, false>);
        } else if (x_dtype == LFFN_BF16) {
            kern = wide ? (x0 ? hash_block64_kernel<__nv_bfloat16, 512, true> : hash_block64_kernel<__nv_bfloat16, 512, false>)
                        : (x0 ? hash_block64_kernel<__nv_bfloat16, 256, true> : hash_block64_kernel<__nv_bfloat16, 256, false>);
        } else {
            set_error("hash_fwd: unknown x dtype %d", x_dtype);
            return LFFN_ERR_INVALID_ARG;
        }
        LFFN_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_k));
        kern<<<(unsigned)grid, threads, smem_k, st>>>(a);
        LFFN_CHECK_CUDA(cudaGetLastError());
        return LFFN_OK;
    }
    if (x_dtype == LFFN_F32) {
        auto kern = hash_block_kernel<float>;
        LFFN_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kern<<<(unsigned)grid, HB_THREADS, smem, st>>>(a, BS, transpose_w);
    } else if (x_dtype == LFFN_BF16) {
        auto kern = hash_block_kernel<__nv_bfloat16>;
        LFFN_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kern<<<(unsigned)grid, HB_THREADS, smem, st>>>(a, BS, transpose_w);
    } else {
        set_error("hash_fwd: unknown x dtype %d", x_dtype);
        return LFFN_ERR_INVALID_ARG;
    }
    LFFN_CHECK_CUDA(cudaGetLastError());
    return LFFN_OK;
}

}  // namespace lffn

#ifdef LFFN_HB_PHASE_CLOCKS
// Reads (and optionally clears) the phase counters of hash_block64_kernel: cycles summed over CTAs, indexed by HB_PH_*.
extern "C" int lffn_debug_hash_block_phases(unsigned long long *out8, int reset) {
    if (out8 != nullptr && cudaMemcpyFromSymbol(out8, lffn::g_hb_phase, 8 * sizeof(unsigned long long)) != cudaSuccess) return -3;
    if (reset) {
        const unsigned long long zero[8] = {0};
        if (cudaMemcpyToSymbol(lffn::g_hb_phase, zero, sizeof(zero)) != cudaSuccess) return -3;
    }
    return 0;
}
#endif
