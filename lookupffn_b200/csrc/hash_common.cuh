// Pieces shared by the two hashing kernels (hash_fwd.cu: diagonal projection, one warp per token;
// hash_block.cu: block-diagonal projection, one CTA per 32-token tile).
#pragma once

#include "common.cuh"

namespace lffn {

struct HashArgs {
    const void *x;
    long long N;
    int d_in, D, S, R;
    int r_lo, r_hi;  // rotations needed for the requested tables, inclusive
    float had_scale, mix_a, mix_b;
    const float *w;     // [R, S, D]
    const float *bias;  // [T*k] or null
    int T, k, bit_order, weight_mode;
    float tau;
    int t_begin, t_count;
    int32_t *idx_out;  // may be null together with w_out: only z_out is produced
    float *w_out;
    float *z_out;
    uint32_t *status;  // device status word (may be null)
    // optional LayerNorm prologue (lookup.py:84,99): u = (x - mean) * rstd * ln_g + ln_b over the d_in columns,
    // biased variance, eps inside the square root; ln_g == nullptr: x is used as it is
    const float *ln_g;
    const float *ln_b;
    float ln_eps;
    // training's backward pass through a block-diagonal projection (hash_block64_kernel modes 1 and 2, proj_bwd.cu)
    float *act_out;    // [S][tiles][D][32]: stage inputs (mode 1) or transformed stage-output gradients (mode 2)
    const float *dz;   // mode 2: upstream gradient [N, dz_cols]
    int dz_cols;
    float *du_out;     // mode 2: gradient with respect to the rotation's input, [tiles][D][32]
};

// LayerNorm statistics of one row held by a warp: `sum` and then `sq` are this lane's partial sums.
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) v += __shfl_xor_sync(FULL, v, s);
    return v;
}
__device__ __forceinline__ float ln_apply(float x, float mean, float rstd, float g, float b) {
    return __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(x, mean), rstd), g), b);
}

// e^x for x <= 0 as one multiply and one ex2.approx.  The result is only ever used as 1 + e^x: its error (about two
// ulp of e^x, plus |x| * 2^-24 relative from rounding x * log2(e), which matters only where e^x is tiny) moves
// 1 + e^x by no more than the two-ulp bound of the library expf does, at a quarter of the instructions.
__device__ __forceinline__ float exp_nonpos(float x) { return __expf(x); }

// ---- a token's row spread over a warp: coordinate e = j * 32 + lane in register j ("scalar layout") ----------------
template <int V, typename XT>
__device__ __forceinline__ void load_row(float (&v)[V], const XT *row, int d_in, int lane) {
#pragma unroll
    for (int j = 0; j < V; j++) {
        const int e = j * 32 + lane;
        v[j] = e < d_in ? Elem<XT>::load1(row + e) : 0.f;
    }
}

// mean and 1/sqrt(var + eps) of a row spread over a warp as in load_row (two passes over the registers)
template <int V>
__device__ __forceinline__ void row_stats(const float (&v)[V], int d_in, int lane, float eps, float &mean, float &rstd) {
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < V; j++) s += v[j];  // padding columns hold zeros
    mean = warp_sum(s) / (float)d_in;
    float q = 0.f;
#pragma unroll
    for (int j = 0; j < V; j++) {
        const float c = (j * 32 + lane < d_in) ? v[j] - mean : 0.f;
        q = fmaf(c, c, q);
    }
    rstd = 1.f / sqrtf(warp_sum(q) / (float)d_in + eps);
}

template <int V>
__device__ __forceinline__ void row_normalise(float (&v)[V], int d_in, int lane, float mean, float rstd,
                                              const float *__restrict__ g, const float *__restrict__ b) {
#pragma unroll
    for (int j = 0; j < V; j++) {
        const int e = j * 32 + lane;
        if (e < d_in) v[j] = ln_apply(v[j], mean, rstd, __ldg(g + e), b != nullptr ? __ldg(b + e) : 0.f);
    }
}

// the kernel of hash_diag_t.cu; returns false when the request is outside what it covers
bool try_launch_hash_transposing(const HashArgs &a, int x_dtype, cudaStream_t st, int *rc);

// ---- codes and weights of one table from its k coordinates ------------------------------------
// `get(j)` returns coordinate j of the table.  Writes m = 1 or k+1 (idx, w) pairs.
template <typename Get>
__device__ __forceinline__ void emit_table(Get get, int k, int bit_order, int weight_mode, float tau, int32_t offset,
                                           bool have_code, int32_t code_lsb, int32_t *io, float *wo) {
    int32_t code = 0;
    if (weight_mode == LFFN_WEIGHT_SCORE) {
        float num = 0.f, den = 1.f;
        for (int j = 0; j < k; j++) {
            const float z = get(j);
            if (!have_code && z > 0.f) code |= 1 << j;
            const float a = fabsf(z);
            num = __fadd_rn(num, a);
            den = __fmul_rn(den, __fadd_rn(1.f, exp_nonpos(__fmul_rn(-2.f, a))));
        }
        if (have_code) code = code_lsb;
        if (bit_order == LFFN_BIT_MSB_FIRST) code = (int32_t)(__brev((unsigned)code) >> (32 - k));
        io[0] = code + offset;
        wo[0] = __fdiv_rn(num, den);
    } else if (weight_mode == LFFN_WEIGHT_ONES) {
        if (have_code) {
            code = code_lsb;
        } else {
            for (int j = 0; j < k; j++)
                if (get(j) > 0.f) code |= 1 << j;
        }
        if (bit_order == LFFN_BIT_MSB_FIRST) code = (int32_t)(__brev((unsigned)code) >> (32 - k));
        io[0] = code + offset;
        wo[0] = 1.f;
    } else {  // soft flip: k+1 candidates
        float s[16];
#pragma unroll
        for (int j = 0; j < 16; j++) {
            if (j < k) {
                const float z = get(j);
                if (!have_code && z > 0.f) code |= 1 << j;
                s[j] = __fdiv_rn(1.f, __fadd_rn(1.f, exp_nonpos(__fdiv_rn(-fabsf(z), tau))));
            }
        }
        if (have_code) code = code_lsb;
        for (int c = 0; c <= k; c++) {
            float p = 1.f;
#pragma unroll
            for (int j = 0; j < 16; j++)
                if (j < k) p = __fmul_rn(p, (c == j + 1) ? __fsub_rn(1.f, s[j]) : s[j]);
            int32_t cc = c == 0 ? code : (code ^ (1 << (c - 1)));
            if (bit_order == LFFN_BIT_MSB_FIRST) cc = (int32_t)(__brev((unsigned)cc) >> (32 - k));
            io[c] = cc + offset;
            wo[c] = p;
        }
    }
}

// The same arithmetic for a table whose K coordinates sit in registers (compile-time K, fully
// unrolled so that the register array is indexed statically).  Operation order = emit_table.
template <int K>
__device__ __forceinline__ void emit_table_regs(const float (&z)[8], int sub, int bit_order, int weight_mode, float tau,
                                                int32_t offset, int32_t *io, float *wo) {
    int32_t code = 0;
    float zz[K];
#pragma unroll
    for (int j = 0; j < K; j++) {
        float t = 0.f;
#pragma unroll
        for (int s = 0; s < 8 / K; s++)
            if (s == sub) t = z[s * K + j];
        zz[j] = t;
        if (t > 0.f) code |= 1 << j;
    }
    if (weight_mode == LFFN_WEIGHT_SCORE) {
        float num = 0.f, den = 1.f;
#pragma unroll
        for (int j = 0; j < K; j++) {
            const float a = fabsf(zz[j]);
            num = __fadd_rn(num, a);
            den = __fmul_rn(den, __fadd_rn(1.f, exp_nonpos(__fmul_rn(-2.f, a))));
        }
        if (bit_order == LFFN_BIT_MSB_FIRST) code = (int32_t)(__brev((unsigned)code) >> (32 - K));
        io[0] = code + offset;
        wo[0] = __fdiv_rn(num, den);
    } else if (weight_mode == LFFN_WEIGHT_ONES) {
        if (bit_order == LFFN_BIT_MSB_FIRST) code = (int32_t)(__brev((unsigned)code) >> (32 - K));
        io[0] = code + offset;
        wo[0] = 1.f;
    } else {
        float s[K];
#pragma unroll
        for (int j = 0; j < K; j++) s[j] = __fdiv_rn(1.f, __fadd_rn(1.f, exp_nonpos(__fdiv_rn(-fabsf(zz[j]), tau))));
#pragma unroll
        for (int c = 0; c <= K; c++) {
            float p = 1.f;
#pragma unroll
            for (int j = 0; j < K; j++) p = __fmul_rn(p, (c == j + 1) ? __fsub_rn(1.f, s[j]) : s[j]);
            int32_t cc = c == 0 ? code : (code ^ (1 << (c - 1)));
            if (bit_order == LFFN_BIT_MSB_FIRST) cc = (int32_t)(__brev((unsigned)cc) >> (32 - K));
            io[c] = cc + offset;
            wo[c] = p;
        }
    }
}

}  // namespace lffn
