// Backward pass of the block-diagonal (BH4) projection: the reference trains through it with autograd over
// torch.einsum and its Hadamard kernel (bh4/kernel.py:23-36, bh4/fast_hadamard_transform/kernel.py:47-54).
//
//   forward, per rotation r:  y_0 = u (x zero-padded);  t_s = blockdiag(W[r,s]) y_s;  y_{s+1} = H t_s * had_scale
//                             z = mix_a * concat_r y_S + mix_b * tile(u) (first T*k columns) + bias
//   backward from dz:         g_S = mix_a * dz_r;  for s = S-1 .. 0:  gt_s = H g_{s+1} * had_scale   (H is symmetric)
//                                 dW[r,s][nb][o][i] = sum_n gt_s[n, nb*64+o] * y_s[n, nb*64+i]
//                                 g_s[n, nb*64+i]   = sum_o gt_s[n, nb*64+o] * W[r,s][nb][o][i]
//                             du = sum_r g_0^r + mix_b * sum_r dz_r;   dbias = sum_n dz
//
// Per rotation, four launches on the caller's stream:
//   1. hash_block64_kernel mode 1: the forward walk again, saving y_0 .. y_{S-1} per 32-token tile
//   2. hash_block64_kernel mode 2: the backward walk, saving gt_s per tile and g_0
//   3. proj_dw_partial_kernel: for every (s, block) the 64 x 64 sum over tokens of gt_s (x) y_s, split over token
//      ranges into partial sums; proj_dw_reduce_kernel adds the partials in a fixed order (deterministic)
//   4. proj_du_kernel: g_0 back to row-major, accumulated over the rotations, plus the mix_b term
// and proj_dbias_partial_kernel + the same fixed-order reduce for the bias gradient.  All fp32 FMA, no tensor cores, no atomics.
#include "common.cuh"
#include "hash_common.cuh"

namespace lffn {

int launch_hash_block64_mode(const HashArgs &a, int mode, int x_dtype, cudaStream_t st);  // hash_block.cu

constexpr int TILE_M = 32;       // tokens per tile of the saved activations: [D][32] floats per tile
constexpr int DW_THREADS = 128;  // one 8 (o) x 4 (i) register tile of the 64 x 64 block per thread
constexpr int DW_LD = 64;        // row length of the transposed [token][64] staging arrays
// The staging arrays are swizzled instead of padded: the 4-float chunk c of token row m sits at chunk position
// c ^ ((m >> 2) & 7).  The transposing 4-byte stores of a warp (eight token quads x four coordinates of one chunk) then
// fall into 32 different banks, and the 16-byte loads of the arithmetic still touch whole, differently ordered chunks
// of a row.  (With padded rows those stores were four-way bank conflicts and the kernel was bound by shared-memory
// bandwidth: 82 % of its peak, a quarter of the wavefronts being conflicts.)
__device__ __forceinline__ int dw_addr(int m, int e) { return m * DW_LD + ((((e >> 2) ^ ((m >> 2) & 7)) << 2) | (e & 3)); }

// grid: x = s * NB + nb, y = split.  acts_g / acts_y: [S][ntiles][D][32].
__global__ void __launch_bounds__(DW_THREADS) proj_dw_partial_kernel(const float *__restrict__ acts_g,
                                                                    const float *__restrict__ acts_y, float *__restrict__ partial,
                                                                    long long ntiles, int D, int splits) {
    __shared__ __align__(16) float Gs[2][TILE_M * DW_LD];
    __shared__ __align__(16) float Ys[2][TILE_M * DW_LD];
    const int NB = D / 64;
    const int s = blockIdx.x / NB, nb = blockIdx.x % NB, split = blockIdx.y;
    const long long t_lo = ntiles * split / splits, t_hi = ntiles * (split + 1) / splits;
    const int tid = threadIdx.x;
    const int to = tid >> 4, ti = tid & 15;  // o0 = 8 * to, i0 = 4 * ti
    const size_t tile_floats = (size_t)D * TILE_M;
    const float *gbase = acts_g + (size_t)s * ntiles * tile_floats + (size_t)nb * 64 * TILE_M;
    const float *ybase = acts_y + (size_t)s * ntiles * tile_floats + (size_t)nb * 64 * TILE_M;
    float acc[8][4];
#pragma unroll
    for (int p = 0; p < 8; p++)
#pragma unroll
        for (int q = 0; q < 4; q++) acc[p][q] = 0.f;

    // a (tile, block) chunk is 64 coordinates x 32 tokens = 2048 contiguous floats: four float4 per thread and array
    float4 rg[4], ry[4];
    auto fetch = [&](long long t) {
        const float4 *gp = reinterpret_cast<const float4 *>(gbase + (size_t)t * tile_floats);
        const float4 *yp = reinterpret_cast<const float4 *>(ybase + (size_t)t * tile_floats);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            rg[j] = __ldg(gp + tid + j * DW_THREADS);
            ry[j] = __ldg(yp + tid + j * DW_THREADS);
        }
    };
    auto stage = [&](int b) {  // registers -> shared memory, transposed to [token][coordinate]
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int f = (tid + j * DW_THREADS) * 4;  // float index in the chunk: e = f / 32, m = f % 32 .. +3
            const int e = f >> 5, m = f & 31;
            const int a0 = dw_addr(m, e);  // m is a multiple of 4: the four rows share the swizzle
            Gs[b][a0] = rg[j].x; Gs[b][a0 + DW_LD] = rg[j].y;
            Gs[b][a0 + 2 * DW_LD] = rg[j].z; Gs[b][a0 + 3 * DW_LD] = rg[j].w;
            Ys[b][a0] = ry[j].x; Ys[b][a0 + DW_LD] = ry[j].y;
            Ys[b][a0 + 2 * DW_LD] = ry[j].z; Ys[b][a0 + 3 * DW_LD] = ry[j].w;
        }
    };
    if (t_lo < t_hi) {
        fetch(t_lo);
        stage(0);
    }
    __syncthreads();
    int b = 0;
    for (long long t = t_lo; t < t_hi; t++, b ^= 1) {
        if (t + 1 < t_hi) fetch(t + 1);  // in flight during the arithmetic below
        const float *G = Gs[b], *Yv = Ys[b];
#pragma unroll 8
        for (int m = 0; m < TILE_M; m++) {
            const float4 g0 = *reinterpret_cast<const float4 *>(G + dw_addr(m, 8 * to));
            const float4 g1 = *reinterpret_cast<const float4 *>(G + dw_addr(m, 8 * to + 4));
            const float4 y4 = *reinterpret_cast<const float4 *>(Yv + dw_addr(m, 4 * ti));
            const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
            const float yv[4] = {y4.x, y4.y, y4.z, y4.w};
            // two output rows per instruction (packed fused multiply-add: the same fmaf chain per element)
#pragma unroll
            for (int p = 0; p < 8; p += 2)
#pragma unroll
                for (int q = 0; q < 4; q++)
                    fma2(acc[p][q], acc[p + 1][q], gv[p], gv[p + 1], yv[q], yv[q], acc[p][q], acc[p + 1][q]);
        }
        if (t + 1 < t_hi) stage(b ^ 1);  // the other buffer was last read one iteration ago, before the barrier below
        __syncthreads();
    }
    float *out = partial + (((size_t)split * gridDim.x + blockIdx.x) * 64 + 8 * to) * 64 + 4 * ti;
#pragma unroll
    for (int p = 0; p < 8; p++) *reinterpret_cast<float4 *>(out + p * 64) = make_float4(acc[p][0], acc[p][1], acc[p][2], acc[p][3]);
}

// dw[j] = sum over splits of partial[split][j], in split order
__global__ void __launch_bounds__(256) proj_dw_reduce_kernel(const float *__restrict__ partial, float *__restrict__ dw,
                                                            long long n, int splits) {
    for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (long long)gridDim.x * blockDim.x) {
        float v = 0.f;
#pragma unroll 8
        for (int sp = 0; sp < splits; sp++) v += __ldg(partial + (size_t)sp * n + j);
        dw[j] = v;
    }
}

// du[n][e] (+)= g0[tile][e][m] + mix_b * dz[n][r*D + e]; one CTA per tile and 32 coordinates
__global__ void __launch_bounds__(256) proj_du_kernel(const float *__restrict__ g0, const float *__restrict__ dz, int dz_cols,
                                                     float *__restrict__ du, long long N, int D, int r, float mix_b,
                                                     int accumulate) {
    __shared__ float tl[32][33];
    const long long tile = blockIdx.x;
    const int e0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 8 rows of 32
    for (int er = ty; er < 32; er += 8) tl[er][tx] = g0[((size_t)tile * D + e0 + er) * TILE_M + tx];  // [e][m]
    __syncthreads();
    for (int mr = ty; mr < 32; mr += 8) {
        const long long n = tile * TILE_M + mr;
        if (n >= N) continue;
        const int e = e0 + tx;
        float v = tl[tx][mr];
        const long long c = (long long)r * D + e;
        if (mix_b != 0.f && c < dz_cols) v = fmaf(mix_b, __ldg(dz + n * dz_cols + c), v);
        float *o = du + n * D + e;
        *o = accumulate ? *o + v : v;
    }
}

// partial[split][c] = sum over the split's rows of dz[n][c]: 32 columns x one row range per CTA, eight row groups
// summed in a fixed order; proj_dw_reduce_kernel then adds the DBIAS_SPLITS partial rows in split order
constexpr int DBIAS_SPLITS = 64;
__global__ void __launch_bounds__(256) proj_dbias_partial_kernel(const float *__restrict__ dz, float *__restrict__ partial,
                                                                long long N, int cols) {
    __shared__ float part[8][32];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + tx;
    const long long n_lo = N * blockIdx.y / DBIAS_SPLITS, n_hi = N * (blockIdx.y + 1) / DBIAS_SPLITS;
    float v = 0.f;
    if (c < cols)
        for (long long n = n_lo + ty; n < n_hi; n += 8) v += __ldg(dz + n * cols + c);
    part[ty][tx] = v;
    __syncthreads();
    if (ty == 0 && c < cols) {
        float t = 0.f;
        for (int j = 0; j < 8; j++) t += part[j][tx];
        partial[(size_t)blockIdx.y * cols + c] = t;
    }
}

static size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }
static int dw_splits(long long ntiles) {
    long long s = ntiles / 8;  // at least eight tiles per partial sum
    if (s > 32) s = 32;
    if (s < 1) s = 1;
    return (int)s;
}

// workspace: acts_y [S][ntiles][D][32] | acts_g (same) | g0 [ntiles][D][32] | partial [splits][S][NB][64][64]
//            | dbias partial [DBIAS_SPLITS][T*k]
size_t proj_bwd_ws_bytes(int D, int S, int64_t N) {
    const long long ntiles = (N + TILE_M - 1) / TILE_M;
    const size_t tile_bytes = (size_t)D * TILE_M * sizeof(float);
    return 2 * up256((size_t)S * ntiles * tile_bytes) + up256((size_t)ntiles * tile_bytes) +
           up256((size_t)dw_splits(ntiles) * S * (D / 64) * 4096 * sizeof(float));
}
static size_t dbias_ws_bytes(int out_dim) { return up256((size_t)DBIAS_SPLITS * out_dim * sizeof(float)); }

static void fill_args(HashArgs &a, const lffn_hash_desc &h, const void *x, int64_t N) {
    a.x = x;
    a.N = N;
    a.d_in = h.d_in;
    a.D = h.D;
    a.S = h.S;
    a.R = h.R;
    a.had_scale = h.had_scale;
    a.mix_a = h.mix_a;
    a.mix_b = h.mix_b;
    a.bias = nullptr;
    a.T = h.T * h.k;  // every output column its own "table": z [N, T*k]
    a.k = 1;          // no codes here; k = 1 divides every D, which keeps the (tile, rotation) work units independent
    a.bit_order = h.bit_order;
    a.weight_mode = LFFN_WEIGHT_ONES;
    a.tau = h.tau;
    a.t_begin = 0;
    a.t_count = a.T;
    a.idx_out = nullptr;
    a.w_out = nullptr;
    a.z_out = nullptr;
    a.status = status_word();
    a.ln_g = nullptr;
    a.ln_b = nullptr;
    a.ln_eps = 0.f;
    a.act_out = nullptr;
    a.dz = nullptr;
    a.dz_cols = 0;
    a.du_out = nullptr;
}

size_t proj_acts_bytes(int D, int S, int R, int64_t N) {
    const long long ntiles = (N + TILE_M - 1) / TILE_M;
    return (size_t)R * S * ntiles * D * TILE_M * sizeof(float);
}

// training's forward pass: z for all rotations in one launch, every stage's input kept in `acts`
int launch_proj_fwd_train(const lffn_hash_desc &h, const void *x, int x_dtype, int64_t N, float *z, float *acts,
                          cudaStream_t st) {
    HashArgs a;
    fill_args(a, h, x, N);
    a.bias = h.proj_bias;
    a.w = h.proj_w;
    a.r_lo = 0;
    a.r_hi = h.R - 1;  // every rotation the backward pass will walk
    a.z_out = z;
    a.act_out = acts;
    return launch_hash_block64_mode(a, 1, x_dtype, st);
}

int launch_proj_bwd(const lffn_hash_desc &h, const float *w_oi, const void *x, int x_dtype, int64_t N, const float *dz,
                    float *du, float *dw, float *dbias, const float *saved_acts, void *ws, cudaStream_t st) {
    const int D = h.D, S = h.S, NB = D / 64;
    const long long ntiles = (N + TILE_M - 1) / TILE_M;
    const size_t tile_bytes = (size_t)D * TILE_M * sizeof(float);
    char *p = static_cast<char *>(ws);
    float *acts_y = reinterpret_cast<float *>(p);
    p += up256((size_t)S * ntiles * tile_bytes);
    float *acts_g = reinterpret_cast<float *>(p);
    p += up256((size_t)S * ntiles * tile_bytes);
    float *g0 = reinterpret_cast<float *>(p);
    p += up256((size_t)ntiles * tile_bytes);
    float *partial = reinterpret_cast<float *>(p);
    const int splits = dw_splits(ntiles);
    const int out_dim = h.T * h.k;
    p += up256((size_t)splits * S * NB * 4096 * sizeof(float));
    float *dbias_partial = reinterpret_cast<float *>(p);

    HashArgs a;
    fill_args(a, h, x, N);
    a.dz = dz;
    a.dz_cols = out_dim;
    a.du_out = g0;
    const size_t rot_floats = (size_t)S * ntiles * D * TILE_M;
    for (int r = 0; r < h.R; r++) {
        a.r_lo = a.r_hi = r;
        int rc = LFFN_OK;
        const float *ys = acts_y;
        if (saved_acts != nullptr) {
            ys = saved_acts + (size_t)r * rot_floats;  // kept by the forward pass
        } else {
            a.w = h.proj_w;  // [i][o]: input-major for the forward product
            a.act_out = acts_y;
            rc = launch_hash_block64_mode(a, 1, x_dtype, st);
            if (rc != LFFN_OK) return rc;
        }
        a.w = w_oi;  // [o][i]: input-major for the backward product
        a.act_out = acts_g;
        rc = launch_hash_block64_mode(a, 2, x_dtype, st);
        if (rc != LFFN_OK) return rc;
        if (dw != nullptr) {
            proj_dw_partial_kernel<<<dim3(S * NB, splits), DW_THREADS, 0, st>>>(acts_g, ys, partial, ntiles, D, splits);
            LFFN_CHECK_CUDA(cudaGetLastError());
            const long long n = (long long)S * NB * 4096;
            proj_dw_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(partial, dw + (size_t)r * n, n, splits);
            LFFN_CHECK_CUDA(cudaGetLastError());
        }
        if (du != nullptr) {
            proj_du_kernel<<<dim3((unsigned)ntiles, D / 32), 256, 0, st>>>(g0, dz, out_dim, du, N, D, r, h.mix_b, r > 0 ? 1 : 0);
            LFFN_CHECK_CUDA(cudaGetLastError());
        }
    }
    if (dbias != nullptr) {
        proj_dbias_partial_kernel<<<dim3((out_dim + 31) / 32, DBIAS_SPLITS), 256, 0, st>>>(dz, dbias_partial, N, out_dim);
        LFFN_CHECK_CUDA(cudaGetLastError());
        proj_dw_reduce_kernel<<<(out_dim + 255) / 256, 256, 0, st>>>(dbias_partial, dbias, out_dim, DBIAS_SPLITS);
        LFFN_CHECK_CUDA(cudaGetLastError());
    }
    return LFFN_OK;
}

}  // namespace lffn

using namespace lffn;

extern "C" size_t lffn_proj_bwd_ws_bytes(const lffn_hash_desc *desc, int64_t N) {
    if (desc == nullptr || N < 1 || desc->BS != 64 || desc->D % 256 != 0 || desc->S < 1) return 0;
    return proj_bwd_ws_bytes(desc->D, desc->S, N) + dbias_ws_bytes(desc->T * desc->k);
}

static int check_proj_desc(const lffn_hash_desc *desc, const char *who) {
    LFFN_REQUIRE(desc != nullptr && desc->proj_w != nullptr, LFFN_ERR_INVALID_ARG, "%s: NULL descriptor or weights", who);
    LFFN_REQUIRE(desc->BS == 64 && desc->transpose_w == 1 && desc->D % 256 == 0 && desc->D >= 256 && desc->D <= 1024,
                 LFFN_ERR_UNSUPPORTED,
                 "%s: covers 64 x 64 blocks with D in {256, 512, 1024} and desc->proj_w in [i][o] order "
                 "(transpose_w = 1); got BS = %d, D = %d, transpose_w = %d", who, desc->BS, desc->D, desc->transpose_w);
    LFFN_REQUIRE(desc->d_in >= 1 && desc->d_in <= desc->D && desc->S >= 1 && desc->R >= 1 && desc->T >= 1 && desc->k >= 1 &&
                     (long long)desc->R * desc->D >= (long long)desc->T * desc->k,
                 LFFN_ERR_INVALID_ARG, "%s: inconsistent descriptor", who);
    return LFFN_OK;
}

extern "C" size_t lffn_proj_acts_bytes(const lffn_hash_desc *desc, int64_t N) {
    if (desc == nullptr || N < 1 || desc->BS != 64 || desc->D % 256 != 0 || desc->S < 1 || desc->R < 1) return 0;
    return proj_acts_bytes(desc->D, desc->S, desc->R, N);
}

extern "C" int lffn_proj_fwd_train(const lffn_hash_desc *desc, const void *x, int32_t x_dtype, int64_t N, float *z,
                                   float *acts, size_t acts_bytes, lffn_stream_t stream) {
    int rc = check_proj_desc(desc, "proj_fwd_train");
    if (rc != LFFN_OK) return rc;
    LFFN_REQUIRE(N >= 0, LFFN_ERR_INVALID_ARG, "proj_fwd_train: N = %lld", (long long)N);
    if (N == 0) return LFFN_OK;
    LFFN_REQUIRE(x != nullptr && z != nullptr && acts != nullptr, LFFN_ERR_INVALID_ARG, "proj_fwd_train: NULL buffer");
    LFFN_REQUIRE(acts_bytes >= proj_acts_bytes(desc->D, desc->S, desc->R, N), LFFN_ERR_SCRATCH,
                 "proj_fwd_train: %zu bytes needed for the stage inputs, %zu given",
                 proj_acts_bytes(desc->D, desc->S, desc->R, N), acts_bytes);
    return launch_proj_fwd_train(*desc, x, x_dtype, N, z, acts, static_cast<cudaStream_t>(stream));
}

extern "C" int lffn_proj_bwd(const lffn_hash_desc *desc, const float *proj_w_oi, const void *x, int32_t x_dtype, int64_t N,
                             const float *dz, float *du, float *dw, float *dbias, const float *saved_acts, void *ws,
                             size_t ws_bytes, lffn_stream_t stream) {
    int rcd = check_proj_desc(desc, "proj_bwd");
    if (rcd != LFFN_OK) return rcd;
    LFFN_REQUIRE(proj_w_oi != nullptr, LFFN_ERR_INVALID_ARG, "proj_bwd: NULL weights");
    LFFN_REQUIRE(N >= 0, LFFN_ERR_INVALID_ARG, "proj_bwd: N = %lld", (long long)N);
    if (N == 0) return LFFN_OK;
    LFFN_REQUIRE(x != nullptr && dz != nullptr && ws != nullptr, LFFN_ERR_INVALID_ARG, "proj_bwd: NULL buffer");
    const size_t need = proj_bwd_ws_bytes(desc->D, desc->S, N) + dbias_ws_bytes(desc->T * desc->k);
    LFFN_REQUIRE(ws_bytes >= need, LFFN_ERR_SCRATCH, "proj_bwd: workspace of %zu bytes needed, %zu given", need, ws_bytes);
    LFFN_REQUIRE((reinterpret_cast<uintptr_t>(ws) & 255u) == 0 && (reinterpret_cast<uintptr_t>(proj_w_oi) & 15u) == 0,
                 LFFN_ERR_INVALID_ARG, "proj_bwd: ws must be 256-byte aligned, the weights 16-byte aligned");
    return launch_proj_bwd(*desc, proj_w_oi, x, x_dtype, N, dz, du, dw, dbias, saved_acts, ws,
                           static_cast<cudaStream_t>(stream));
}

// Gradient of a bias that was added to every row: out[c] = sum_n dy[n][c], the two kernels of the projection's bias
// gradient (partial sums over 64 row ranges, added in range order: deterministic).  Replaces the reduction autograd
// runs for `outputs + self.bias` (lookup.py:108).  ws: lffn_bias_grad_ws_bytes(cols) bytes.
extern "C" size_t lffn_bias_grad_ws_bytes(int32_t cols) { return dbias_ws_bytes(cols); }

extern "C" int lffn_bias_grad(const float *dy, int64_t N, int32_t cols, float *dbias, void *ws, size_t ws_bytes,
                              lffn_stream_t stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    LFFN_REQUIRE(dy != nullptr && dbias != nullptr && N >= 0 && cols > 0, LFFN_ERR_INVALID_ARG, "bias_grad: bad argument");
    LFFN_REQUIRE(ws != nullptr && ws_bytes >= dbias_ws_bytes(cols), LFFN_ERR_SCRATCH, "bias_grad: workspace of %zu bytes needed",
                 dbias_ws_bytes(cols));
    float *partial = static_cast<float *>(ws);
    proj_dbias_partial_kernel<<<dim3((cols + 31) / 32, DBIAS_SPLITS), 256, 0, st>>>(dy, partial, N, cols);
    LFFN_CHECK_CUDA(cudaGetLastError());
    proj_dw_reduce_kernel<<<(cols + 255) / 256, 256, 0, st>>>(partial, dbias, cols, DBIAS_SPLITS);
    LFFN_CHECK_CUDA(cudaGetLastError());
    return LFFN_OK;
}
