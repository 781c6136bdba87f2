// Backward of the layer's LayerNorm (lookup.py:84,99: torch.nn.LayerNorm over the hidden dimension, biased variance,
// eps inside the square root), the last piece of the layer's backward pass:
//   xhat = (x - mean) * rstd,  u = xhat * gamma + beta
//   g = du * gamma,  dx = rstd * (g - mean(g) - xhat * mean(g * xhat))
//   dgamma = sum_n du * xhat,  dbeta = sum_n du
// One warp owns a row at a time (x, du in registers, coordinate e = j * 32 + lane) and recomputes the statistics
// the way the forward kernels do; every warp keeps its own column sums for dgamma / dbeta in registers, the warps of
// a CTA add theirs in warp order, and a second kernel adds the CTAs' partial rows in CTA order: no atomics, the same
// bits on every run.
#include "common.cuh"
#include "hash_common.cuh"

namespace lffn {

constexpr int LNB_WARPS = 8;

template <int V>
__global__ void __launch_bounds__(LNB_WARPS * 32) layernorm_bwd_kernel(const float *__restrict__ x, const float *__restrict__ du,
                                                                       const float *__restrict__ gamma, long long N, float eps,
                                                                       float *__restrict__ dx, float *__restrict__ partial) {
    constexpr int d = V * 32;
    extern __shared__ float comb[];  // [LNB_WARPS][2 d]: every warp's column sums (dgamma row, then dbeta row)
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const long long warp0 = (long long)blockIdx.x * LNB_WARPS + wib, nwarps = (long long)gridDim.x * LNB_WARPS;
    float gm[V], ag[V], ab[V];
#pragma unroll
    for (int j = 0; j < V; j++) {
        gm[j] = __ldg(gamma + j * 32 + lane);
        ag[j] = 0.f;
        ab[j] = 0.f;
    }
    for (long long n = warp0; n < N; n += nwarps) {
        float xv[V], dv[V];
#pragma unroll
        for (int j = 0; j < V; j++) {
            xv[j] = __ldg(x + n * d + j * 32 + lane);
            dv[j] = __ldg(du + n * d + j * 32 + lane);
        }
        float mean, rstd;
        row_stats<V>(xv, d, lane, eps, mean, rstd);
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int j = 0; j < V; j++) {
            xv[j] = (xv[j] - mean) * rstd;  // xhat
            const float g = dv[j] * gm[j];
            s1 += g;
            s2 = fmaf(g, xv[j], s2);
            ag[j] = fmaf(dv[j], xv[j], ag[j]);
            ab[j] += dv[j];
        }
        s1 = warp_sum(s1) / (float)d;
        s2 = warp_sum(s2) / (float)d;
#pragma unroll
        for (int j = 0; j < V; j++) dx[n * d + j * 32 + lane] = rstd * (dv[j] * gm[j] - s1 - xv[j] * s2);
    }
#pragma unroll
    for (int j = 0; j < V; j++) {
        comb[wib * 2 * d + j * 32 + lane] = ag[j];
        comb[wib * 2 * d + d + j * 32 + lane] = ab[j];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * d; i += LNB_WARPS * 32) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < LNB_WARPS; w++) t += comb[w * 2 * d + i];
        partial[(size_t)blockIdx.x * 2 * d + i] = t;
    }
}

// out[i] = sum over the CTAs' partial rows, i in [0, 2d): dgamma then dbeta.  32 columns x 8 groups per CTA: group g
// adds rows g, g + 8, ... in order, then the eight group sums are added in group order (fixed order, short chains).
__global__ void __launch_bounds__(256) layernorm_bwd_reduce_kernel(const float *__restrict__ partial, float *__restrict__ dgamma,
                                                                   float *__restrict__ dbeta, int d, int blocks) {
    __shared__ float part[8][32];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int i = blockIdx.x * 32 + tx;
    float t = 0.f;
    if (i < 2 * d)
        for (int b = ty; b < blocks; b += 8) t += __ldg(partial + (size_t)b * 2 * d + i);
    part[ty][tx] = t;
    __syncthreads();
    if (ty == 0 && i < 2 * d) {
        float v = 0.f;
#pragma unroll
        for (int g = 0; g < 8; g++) v += part[g][tx];
        if (i < d) dgamma[i] = v;
        else dbeta[i - d] = v;
    }
}

static int ln_bwd_blocks() { return 2 * num_sms(); }

}  // namespace lffn

using namespace lffn;

extern "C" size_t lffn_layernorm_bwd_ws_bytes(int32_t d) { return (size_t)ln_bwd_blocks() * 2 * (size_t)d * sizeof(float); }

extern "C" int lffn_layernorm_bwd(const float *x, const float *du, const float *gamma, int64_t N, int32_t d, float eps,
                                  float *dx, float *dgamma, float *dbeta, void *ws, size_t ws_bytes, lffn_stream_t stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    LFFN_REQUIRE(x != nullptr && du != nullptr && gamma != nullptr && dx != nullptr && dgamma != nullptr && dbeta != nullptr,
                 LFFN_ERR_INVALID_ARG, "layernorm_bwd: null argument");
    LFFN_REQUIRE(N >= 0 && (d == 256 || d == 512 || d == 768 || d == 1024), LFFN_ERR_UNSUPPORTED,
                 "layernorm_bwd: hidden size %d unsupported (256, 512, 768 or 1024)", d);
    LFFN_REQUIRE(ws != nullptr && ws_bytes >= lffn_layernorm_bwd_ws_bytes(d), LFFN_ERR_SCRATCH,
                 "layernorm_bwd: workspace of %zu bytes needed", lffn_layernorm_bwd_ws_bytes(d));
    const int blocks = ln_bwd_blocks();
    float *partial = static_cast<float *>(ws);
    const size_t smem = (size_t)LNB_WARPS * 2 * d * sizeof(float);
    void (*kern)(const float *, const float *, const float *, long long, float, float *, float *) =
        d == 256 ? layernorm_bwd_kernel<8> : d == 512 ? layernorm_bwd_kernel<16> : d == 768 ? layernorm_bwd_kernel<24> : layernorm_bwd_kernel<32>;
    if (smem > 48 * 1024) LFFN_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<blocks, LNB_WARPS * 32, smem, st>>>(x, du, gamma, N, eps, dx, partial);
    LFFN_CHECK_CUDA(cudaGetLastError());
    layernorm_bwd_reduce_kernel<<<(2 * d + 31) / 32, 256, 0, st>>>(partial, dgamma, dbeta, d, blocks);
    LFFN_CHECK_CUDA(cudaGetLastError());
    return LFFN_OK;
}
