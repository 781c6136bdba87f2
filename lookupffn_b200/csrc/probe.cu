// Measurement probe: how fast can coalesced 16-byte read-only loads that do not allocate in L1 -- the gather's
// row loads -- pull bytes that are resident in L2?  The answer depends on how many bytes an SM keeps in flight
// (loads in flight per thread x resident warps), so the probe has three configurations and the benchmark quotes
// the gather against the best of them:
//   mode 0: 12 loads in flight per thread, 4 CTAs of 128 threads per SM -- the gather kernel's own residency
//   mode 1:  8 loads in flight per thread, as many CTAs per SM as fit
//   mode 2: 16 loads in flight per thread, as many CTAs per SM as fit
//   mode 3:  4 loads in flight per thread, 16 CTAs per SM (all 64 warps resident)
// It runs outside the benchmark's timed region.  No reference counterpart; nothing on the layer's path calls it.
#include "common.cuh"

namespace lffn {

constexpr int PROBE_THREADS = 128;

template <int IN_FLIGHT, int MINBLOCKS>
__global__ void __launch_bounds__(PROBE_THREADS, MINBLOCKS) probe_read_kernel(const uint4 *__restrict__ buf, unsigned iters,
                                                                               int repeats, uint32_t *sink) {
    // The buffer is cut into `iters` slabs of gridDim.x * IN_FLIGHT * PROBE_THREADS vectors; in every slab a CTA
    // reads IN_FLIGHT runs of 128 consecutive vectors (each warp 512 contiguous bytes per load).  No predicates and
    // 32-bit index arithmetic: the loop is loads and two logic instructions per load.
    const unsigned cta_stride = IN_FLIGHT * PROBE_THREADS;
    const unsigned slab = gridDim.x * cta_stride;
    uint32_t x = 0;
    for (int r = 0; r < repeats; r++) {
        const uint4 *p = buf + blockIdx.x * cta_stride + threadIdx.x;
        for (unsigned it = 0; it < iters; it++, p += slab) {
            uint4 v[IN_FLIGHT];
#pragma unroll
            for (int u = 0; u < IN_FLIGHT; u++) v[u] = ld_row16(p + u * PROBE_THREADS);
#pragma unroll
            for (int u = 0; u < IN_FLIGHT; u++) x ^= v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
        }
    }
    if (x == 0x9e3779b9u) *sink = x;  // keeps the loads alive; practically never true
}

// reads the largest whole number of slabs that fits in `bytes`; *bytes_read tells how much that was per repeat
template <int IN_FLIGHT, int MINBLOCKS>
static int launch_probe(const void *buf, size_t bytes, int repeats, uint32_t *sink, int cap_per_sm, size_t *bytes_read,
                        cudaStream_t st) {
    auto kern = probe_read_kernel<IN_FLIGHT, MINBLOCKS>;
    int per_sm = 0;
    LFFN_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, PROBE_THREADS, 0));
    if (per_sm < 1) per_sm = 1;
    if (cap_per_sm > 0 && per_sm > cap_per_sm) per_sm = cap_per_sm;
    const long long grid = (long long)num_sms() * per_sm;
    const size_t slab_bytes = (size_t)grid * IN_FLIGHT * PROBE_THREADS * 16;
    const size_t iters = bytes / slab_bytes;
    LFFN_REQUIRE(iters >= 1 && iters < (1u << 20), LFFN_ERR_INVALID_ARG, "probe_read: %zu bytes are fewer than one slab of %zu",
                 bytes, slab_bytes);
    if (bytes_read != nullptr) *bytes_read = iters * slab_bytes;
    kern<<<(unsigned)grid, PROBE_THREADS, 0, st>>>(static_cast<const uint4 *>(buf), (unsigned)iters, repeats, sink);
    LFFN_CHECK_CUDA(cudaGetLastError());
    return LFFN_OK;
}

int launch_probe_read(const void *buf, size_t bytes, int repeats, int mode, uint32_t *sink, size_t *bytes_read,
                      cudaStream_t st) {
    switch (mode) {
        case 0: return launch_probe<12, 4>(buf, bytes, repeats, sink, 4, bytes_read, st);
        case 1: return launch_probe<8, 8>(buf, bytes, repeats, sink, 0, bytes_read, st);
        case 2: return launch_probe<16, 5>(buf, bytes, repeats, sink, 0, bytes_read, st);
        case 3: return launch_probe<4, 16>(buf, bytes, repeats, sink, 0, bytes_read, st);
    }
    set_error("probe_read: mode %d outside [0, 3]", mode);
    return LFFN_ERR_INVALID_ARG;
}

}  // namespace lffn

extern "C" int lffn_probe_read(const void *buf, size_t bytes, int32_t repeats, int32_t mode, uint32_t *sink,
                               size_t *bytes_read_per_repeat, lffn_stream_t stream) {
    using namespace lffn;
    LFFN_REQUIRE(buf != nullptr && sink != nullptr && bytes >= 16 && repeats >= 1, LFFN_ERR_INVALID_ARG,
                 "probe_read: NULL buffer, fewer than 16 bytes or no repeats");
    LFFN_REQUIRE((reinterpret_cast<uintptr_t>(buf) & 15u) == 0, LFFN_ERR_INVALID_ARG, "probe_read: buf must be 16-byte aligned");
    return launch_probe_read(buf, bytes, repeats, mode, sink, bytes_read_per_repeat, static_cast<cudaStream_t>(stream));
}
