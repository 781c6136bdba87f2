// Measurement probe: how fast can the gather's own access pattern -- coalesced 16-byte read-only loads that do
// not allocate in L1, many of them in flight per thread -- pull bytes that are resident in L2?  The benchmark
// runs it outside its timed region and reports the gather kernel's rate against this ceiling.  No reference
// counterpart; nothing on the layer's path calls it.
#include "common.cuh"

namespace lffn {

constexpr int PROBE_THREADS = 128;
constexpr int PROBE_IN_FLIGHT = 12;  // 16-byte loads in flight per thread, as in the gather's inner loop

__global__ void __launch_bounds__(PROBE_THREADS, 4) probe_read_kernel(const uint4 *__restrict__ buf, long long nvec,
                                                                       int repeats, uint32_t *sink) {
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long nthreads = (long long)gridDim.x * blockDim.x;
    uint32_t x = 0;
    for (int r = 0; r < repeats; r++) {
        // each warp reads 512 contiguous bytes per load; the PROBE_IN_FLIGHT loads of a thread are nthreads apart
        for (long long i = tid; i < nvec; i += nthreads * PROBE_IN_FLIGHT) {
            uint4 v[PROBE_IN_FLIGHT];
#pragma unroll
            for (int u = 0; u < PROBE_IN_FLIGHT; u++) {
                const long long j = i + (long long)u * nthreads;
                v[u] = ld_row16_pred(buf + (j < nvec ? j : 0), j < nvec);
            }
#pragma unroll
            for (int u = 0; u < PROBE_IN_FLIGHT; u++) x ^= v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
        }
    }
    if (x == 0x9e3779b9u) *sink = x;  // keeps the loads alive; practically never true
}

int launch_probe_read(const void *buf, size_t bytes, int repeats, uint32_t *sink, cudaStream_t st) {
    int per_sm = 0;
    LFFN_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, probe_read_kernel, PROBE_THREADS, 0));
    if (per_sm < 1) per_sm = 1;
    if (per_sm > 4) per_sm = 4;  // the gather's residency: 4 CTAs of 128 threads per SM
    const long long grid = (long long)num_sms() * per_sm;
    probe_read_kernel<<<(unsigned)grid, PROBE_THREADS, 0, st>>>(static_cast<const uint4 *>(buf), (long long)(bytes / 16),
                                                               repeats, sink);
    LFFN_CHECK_CUDA(cudaGetLastError());
    return LFFN_OK;
}

}  // namespace lffn

extern "C" int lffn_probe_read(const void *buf, size_t bytes, int32_t repeats, uint32_t *sink, lffn_stream_t stream) {
    using namespace lffn;
    LFFN_REQUIRE(buf != nullptr && sink != nullptr && bytes >= 16 && repeats >= 1, LFFN_ERR_INVALID_ARG,
                 "probe_read: NULL buffer, fewer than 16 bytes or no repeats");
    LFFN_REQUIRE((reinterpret_cast<uintptr_t>(buf) & 15u) == 0, LFFN_ERR_INVALID_ARG, "probe_read: buf must be 16-byte aligned");
    return launch_probe_read(buf, bytes, repeats, sink, static_cast<cudaStream_t>(stream));
}
