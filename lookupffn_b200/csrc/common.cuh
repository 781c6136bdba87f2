// Shared helpers of liblookupffn: error reporting, the device status word, 16-byte vector
// loads/stores and storage-type conversion.  Built for sm_100a only.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/lookupffn.h"

// Long index lists over table sets beyond L2 are consumed in slices of about this many table bytes (gather_fwd.cu,
// gather_bwd.cu): one launch per slice re-aligns the warps along the list.
#ifndef LFFN_GATHER_SLICE_BYTES
#define LFFN_GATHER_SLICE_BYTES 32e6
#endif

namespace lffn {

constexpr unsigned FULL = 0xffffffffu;

// ---- host side -------------------------------------------------------------------------------
void set_error(const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what);
int num_sms();
uint32_t *status_word();  // device pointer to this device's status word (allocated on first use)

#define LFFN_CHECK_CUDA(expr)                                     \
    do {                                                          \
        cudaError_t _e = (expr);                                  \
        if (_e != cudaSuccess) return ::lffn::cuda_fail(_e, #expr); \
    } while (0)

#define LFFN_REQUIRE(cond, code, ...)       \
    do {                                    \
        if (!(cond)) {                      \
            ::lffn::set_error(__VA_ARGS__); \
            return (code);                  \
        }                                   \
    } while (0)

// launchers implemented in the .cu files, called by api.cu after argument checks
int launch_gather_fwd(const int32_t *idx, const float *w, const void *tables, int table_dtype, void *out,
                      int out_dtype, int64_t N, int I, int64_t S, int d, const float *bias, const void *residual,
                      cudaStream_t st);
int launch_gather_fwd_scatter(const int32_t *idx, const float *w, const void *tables, int table_dtype,
                              float *const *peers, long long rows_per_owner, int slab, int first_owner, int64_t N,
                              int I, int64_t S,
                              int d, cudaStream_t st);
int launch_hash_fwd(const lffn_hash_desc &h, const void *x, int x_dtype, int64_t N, int t_begin, int t_count,
                    int32_t *idx_out, float *w_out, float *z_out, const float *ln_g, const float *ln_b, float ln_eps,
                    cudaStream_t st);
int launch_code_weights(const float *z, int64_t N, int T, int k, int bit_order, int weight_mode, float tau,
                        int add_offsets, int32_t *idx_out, float *w_out, cudaStream_t st);
int launch_code_weights_bwd(const float *z, const float *dw, int64_t N, int T, int k, int weight_mode, float tau,
                            float *dz, cudaStream_t st);
int launch_bounded_wait_selftest(int poll_limit, cudaStream_t st);
int launch_fwht(const void *x, void *out, int64_t N, int D, int dtype, float scale, cudaStream_t st);
int launch_gather_bwd_weights(const int32_t *idx, const float *dy, const void *tables, int table_dtype, float *dw,
                              int64_t N, int I, int64_t S, int d, cudaStream_t st);
int launch_gather_bwd_tables(const int32_t *idx, const float *w, const float *dy, float *dtables, int64_t N, int I,
                             int64_t S, int d, cudaStream_t st);
size_t sorted_scratch_bytes(int64_t N, int T, int m, int rows);
int launch_gather_bwd_tables_sorted(const int32_t *idx, const float *w, const float *dy, float *dtables, int64_t N,
                                    int T, int m, int rows, int d, void *scratch, size_t scratch_bytes,
                                    cudaStream_t st);

// ---- device side -----------------------------------------------------------------------------
#ifdef __CUDACC__

// 16-byte read-only load that does not allocate in L1: table rows are touched once per SM.
// Streaming operands (index and weight lists, read once) are loaded with an L2 evict-first policy so that
// they do not push table rows out of L2.
__device__ __forceinline__ unsigned long long policy_evict_first() {
    unsigned long long p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ int ld_stream_i32(const int *p, unsigned long long pol) {
    int v;
    asm volatile("ld.global.nc.L2::cache_hint.s32 %0, [%1], %2;" : "=r"(v) : "l"(p), "l"(pol));
    return v;
}
__device__ __forceinline__ float ld_stream_f32(const float *p, unsigned long long pol) {
    float v;
    asm volatile("ld.global.nc.L2::cache_hint.f32 %0, [%1], %2;" : "=f"(v) : "l"(p), "l"(pol));
    return v;
}

__device__ __forceinline__ uint4 ld_row16(const void *p) {
    uint4 v;
#ifdef LFFN_ROW_LOAD_L1_ALLOCATE
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
#else
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
#endif
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// the same load under a predicate (no branch); returns zeros when the predicate is false
__device__ __forceinline__ uint4 ld_row16_pred(const void *p, bool pred) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    asm volatile(
        "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %5, 0;\n\t"
#ifdef LFFN_ROW_LOAD_L1_ALLOCATE
        "@q ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];\n\t}"
#else
        "@q ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n\t}"
#endif
        : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
        : "l"(p), "r"((int)pred));
    return v;
}

__device__ __forceinline__ float bf16lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

template <typename T>
struct Elem;
template <>
struct Elem<float> {
    static constexpr int PER_VEC = 4;  // elements per 16-byte vector
    static constexpr int DTYPE = LFFN_F32;
    __device__ static __forceinline__ void unpack(const uint4 &v, float (&f)[4]) {
        f[0] = __uint_as_float(v.x);
        f[1] = __uint_as_float(v.y);
        f[2] = __uint_as_float(v.z);
        f[3] = __uint_as_float(v.w);
    }
    __device__ static __forceinline__ float load1(const float *p) { return __ldg(p); }
    __device__ static __forceinline__ void store1(float *p, float v) { *p = v; }
};
template <>
struct Elem<__nv_bfloat16> {
    static constexpr int PER_VEC = 8;
    static constexpr int DTYPE = LFFN_BF16;
    __device__ static __forceinline__ void unpack(const uint4 &v, float (&f)[8]) {
        f[0] = bf16lo(v.x);
        f[1] = bf16hi(v.x);
        f[2] = bf16lo(v.y);
        f[3] = bf16hi(v.y);
        f[4] = bf16lo(v.z);
        f[5] = bf16hi(v.z);
        f[6] = bf16lo(v.w);
        f[7] = bf16hi(v.w);
    }
    __device__ static __forceinline__ float load1(const __nv_bfloat16 *p) {
        return __uint_as_float(((uint32_t) * reinterpret_cast<const unsigned short *>(p)) << 16);
    }
    __device__ static __forceinline__ void store1(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }
};

#endif  // __CUDACC__

}  // namespace lffn
