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
constexpr float LFFN_LOG2E = 1.4426950408889634f;
__device__ __forceinline__ float ex2_approx(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float exp_nonpos(float x) { return ex2_approx(__fmul_rn(x, LFFN_LOG2E)); }

// Packed fp32 arithmetic (add / sub / mul / fma .rn.f32x2): one instruction carries two independent IEEE
// round-to-nearest operations on an aligned register pair, so the results equal the scalar forms bit for bit while
// the instruction count of an issue-bound kernel halves.  Values 2i and 2i+1 of a lane's array form the pairs.
// RULE: the result of mul2 must never feed add2 / sub2 / fma2 directly.  ptxas (12.9) contracts a packed multiply
// and a dependent packed add into one fma.rn.f32x2 although both carry .rn (measured: 17 % of random inputs change
// in the last bit), which would break the two-rounding arithmetic of the CPU oracle.  Scalar __fmul_rn is never
// contracted, so a product that is added afterwards is formed with scalar multiplies and only the add is packed.
#ifndef LFFN_HASH_T_SCALAR
#define LFFN_F32X2_OP(name, op)                                                                                         \
    __device__ __forceinline__ void name(float &r0, float &r1, float a0, float a1, float b0, float b1) {               \
        asm("{ .reg .b64 ra, rb, rc; mov.b64 ra, {%2,%3}; mov.b64 rb, {%4,%5}; " op " rc, ra, rb; mov.b64 {%0,%1}, rc; }" \
            : "=f"(r0), "=f"(r1)                                                                                        \
            : "f"(a0), "f"(a1), "f"(b0), "f"(b1));                                                                      \
    }
LFFN_F32X2_OP(add2, "add.rn.f32x2")
LFFN_F32X2_OP(sub2, "sub.rn.f32x2")
LFFN_F32X2_OP(mul2, "mul.rn.f32x2")
#undef LFFN_F32X2_OP
__device__ __forceinline__ void fma2(float &r0, float &r1, float a0, float a1, float b0, float b1, float c0, float c1) {
    asm("{ .reg .b64 ra, rb, rc, rd; mov.b64 ra, {%2,%3}; mov.b64 rb, {%4,%5}; mov.b64 rc, {%6,%7}; "
        "fma.rn.f32x2 rd, ra, rb, rc; mov.b64 {%0,%1}, rd; }"
        : "=f"(r0), "=f"(r1)
        : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}
#else
__device__ __forceinline__ void add2(float &r0, float &r1, float a0, float a1, float b0, float b1) { r0 = __fadd_rn(a0, b0); r1 = __fadd_rn(a1, b1); }
__device__ __forceinline__ void sub2(float &r0, float &r1, float a0, float a1, float b0, float b1) { r0 = __fsub_rn(a0, b0); r1 = __fsub_rn(a1, b1); }
__device__ __forceinline__ void mul2(float &r0, float &r1, float a0, float a1, float b0, float b1) { r0 = __fmul_rn(a0, b0); r1 = __fmul_rn(a1, b1); }
__device__ __forceinline__ void fma2(float &r0, float &r1, float a0, float a1, float b0, float b1, float c0, float c1) {
    r0 = __fmaf_rn(a0, b0, c0);
    r1 = __fmaf_rn(a1, b1, c1);
}
#endif

// butterfly stages over the register index, strides V/2 down to 1: pairs of butterflies as packed operations while the
// stride keeps both members of a register pair on the same side, scalar for the last stage
template <int V>
__device__ __forceinline__ void reg_butterflies(float (&v)[V]) {
#pragma unroll
    for (int s = V / 2; s >= 2; s >>= 1) {
#pragma unroll
        for (int j = 0; j < V; j += 2) {
            if ((j & s) == 0) {
                const float a0 = v[j], a1 = v[j + 1], b0 = v[j + s], b1 = v[j + s + 1];
                add2(v[j], v[j + 1], a0, a1, b0, b1);
                sub2(v[j + s], v[j + s + 1], a0, a1, b0, b1);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < V; j += 2) {
        const float a = v[j], b = v[j + 1];
        v[j] = __fadd_rn(a, b);
        v[j + 1] = __fsub_rn(a, b);
    }
}

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

// codes and weights of the table whose K coordinates are z[0..K) (registers); operation order = emit_table
template <int K>
__device__ __forceinline__ void emit_table_k(const float *z, int bit_order, int weight_mode, float tau, int32_t offset,
                                             int32_t *io, float *wo) {
    int32_t code = 0;
#pragma unroll
    for (int j = 0; j < K; j++)
        if (z[j] > 0.f) code |= 1 << j;
    if (weight_mode == LFFN_WEIGHT_SCORE) {
        float num = 0.f, den = 1.f;
        if constexpr (K % 2 == 0) {
            // the element-wise part (-2 a, the ex2 prescale, 1 + e) two coordinates per instruction; the sum and the
            // product stay one chain each in coordinate order, like emit_table
#pragma unroll
            for (int j = 0; j < K; j += 2) {
                const float a0 = fabsf(z[j]), a1 = fabsf(z[j + 1]);
                float t0, t1, f0, f1;
                mul2(t0, t1, -2.f, -2.f, a0, a1);
                mul2(t0, t1, t0, t1, LFFN_LOG2E, LFFN_LOG2E);
                add2(f0, f1, 1.f, 1.f, ex2_approx(t0), ex2_approx(t1));
                num = __fadd_rn(__fadd_rn(num, a0), a1);
                den = __fmul_rn(__fmul_rn(den, f0), f1);
            }
        } else {
#pragma unroll
            for (int j = 0; j < K; j++) {
                const float a = fabsf(z[j]);
                num = __fadd_rn(num, a);
                den = __fmul_rn(den, __fadd_rn(1.f, exp_nonpos(__fmul_rn(-2.f, a))));
            }
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
        for (int j = 0; j < K; j++) s[j] = __fdiv_rn(1.f, __fadd_rn(1.f, exp_nonpos(__fdiv_rn(-fabsf(z[j]), tau))));
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
