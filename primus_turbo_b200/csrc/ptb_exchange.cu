// Row-segment copies between GPUs of one node (the expert-parallel dispatch and combine), and the
// MoE row permutation kernels that sit either side of the grouped GEMM.
//
// Dispatch and combine are the same operation: every rank holds rows that are contiguous per
// (destination rank, expert) and knows, from the routing counts of all ranks, the row at which each
// such segment starts in the destination's buffer.  One kernel copies all segments of a rank with plain
// 16-byte loads from local memory and plain 16-byte stores to the destination -- peer memory mapped
// into this process (NVLink / NVSwitch) or local memory for the rank's own share -- so rows land in
// expert-major order, ready for the grouped GEMM, with no staging pass on either side.  The kernel
// waits on nothing; the ranks order themselves with a collective afterwards.
#include "ptb_common.cuh"

namespace ptb {
namespace {

constexpr int kMaxPeers    = 16;
constexpr int kCopyThreads = 512;
constexpr int kChunkBytes  = 4 * kCopyThreads * 16; // 32 KiB per work item: four 16-byte loads in flight per thread
constexpr int kMaxSegments = 8192;

struct CopyArgs {
    const uint8_t *src;
    uint8_t *dst[kMaxPeers];
    const int64_t *segs; // [nseg][4]: first source row, first destination row, rows, destination rank
    int nseg;
    int n_ranks;
    int64_t row_bytes;
};

// set to 1 by a copy whose segment table names a rank outside [0, n_ranks) (that segment is skipped)
__device__ int g_copy_error = 0;

__global__ void __launch_bounds__(kCopyThreads) copy_segments_kernel(const CopyArgs a) {
    // chunk-count prefix over the segments, built by the whole CTA (nseg <= kMaxSegments)
    __shared__ int s_prefix[kMaxSegments + 1];
    __shared__ int s_warp[kCopyThreads / 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int run = 0;
    for (int base = 0; base < a.nseg; base += kCopyThreads) {
        const int s = base + tid;
        int cnt     = 0;
        if (s < a.nseg) cnt = (int) ((a.segs[4 * s + 2] * a.row_bytes + kChunkBytes - 1) / kChunkBytes);
        int inc = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += n;
        }
        if (lane == 31) s_warp[warp] = inc;
        __syncthreads();
        int before = run;
        for (int w = 0; w < warp; ++w) before += s_warp[w];
        if (s < a.nseg) s_prefix[s + 1] = before + inc;
        int total = 0;
        for (int w = 0; w < kCopyThreads / 32; ++w) total += s_warp[w];
        run += total;
        __syncthreads();
    }
    if (tid == 0) s_prefix[0] = 0;
    __syncthreads();
    const int total_chunks = s_prefix[a.nseg];

    for (int c = blockIdx.x; c < total_chunks; c += gridDim.x) {
        // segment that holds chunk c: last s with prefix[s] <= c
        int lo = 0, hi = a.nseg - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (s_prefix[mid] <= c) lo = mid;
            else hi = mid - 1;
        }
        const int64_t *sg = a.segs + 4 * lo;
        const int64_t rank = sg[3];
        if (rank < 0 || rank >= a.n_ranks) {
            if (tid == 0) atomicExch(&g_copy_error, 1);
            continue;
        }
        const int64_t seg_bytes = sg[2] * a.row_bytes;
        const int64_t off       = (int64_t) (c - s_prefix[lo]) * kChunkBytes;
        const int64_t n         = min((int64_t) kChunkBytes, seg_bytes - off);
        const uint4 *src = reinterpret_cast<const uint4 *>(a.src + sg[0] * a.row_bytes + off);
        uint4 *dst       = reinterpret_cast<uint4 *>(a.dst[rank] + sg[1] * a.row_bytes + off);
        const int nvec   = (int) (n >> 4);
        uint4 v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int j = tid + i * kCopyThreads;
            if (j < nvec) v[i] = __ldg(src + j);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int j = tid + i * kCopyThreads;
            if (j < nvec) dst[j] = v[i];
        }
    }
}

// ---- row permutation: out[i] = in[index[i]] (gather) for rows of `row_bytes` bytes -------------------
// One warp per row, 16-byte accesses; rows whose index is negative are written as zeros (dropped tokens).
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint8_t *__restrict__ in, const int64_t *__restrict__ index,
                                                           int64_t n_out, int64_t n_in, int64_t row_bytes,
                                                           uint8_t *__restrict__ out) {
    const int lane  = threadIdx.x & 31;
    const int64_t w = ((int64_t) blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nw = ((int64_t) gridDim.x * blockDim.x) >> 5;
    const int64_t nvec = row_bytes >> 4;
    for (int64_t r = w; r < n_out; r += nw) {
        const int64_t s = index[r];
        uint4 *dst      = reinterpret_cast<uint4 *>(out + r * row_bytes);
        if (s < 0 || s >= n_in) {
            for (int64_t j = lane; j < nvec; j += 32) dst[j] = make_uint4(0, 0, 0, 0);
        } else {
            const uint4 *src = reinterpret_cast<const uint4 *>(in + s * row_bytes);
            for (int64_t j = lane; j < nvec; j += 32) dst[j] = __ldg(src + j);
        }
    }
}

} // namespace
} // namespace ptb

using namespace ptb;

extern "C" {
#pragma GCC visibility push(default)

int ptb_copy_segments(const void *src_base, void *const *dst_bases, int n_ranks, const int64_t *segments, int64_t nseg,
                      int64_t row_bytes, int num_ctas, ptb_stream_t stream) {
    PTB_REQUIRE(n_ranks >= 1 && n_ranks <= kMaxPeers, PTB_ERR_TOO_LARGE, "copy_segments: 1 to %d ranks, got %d", kMaxPeers,
                n_ranks);
    PTB_REQUIRE(nseg >= 0 && nseg <= kMaxSegments, PTB_ERR_TOO_LARGE, "copy_segments: at most %d segments", kMaxSegments);
    PTB_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0, PTB_ERR_ALIGN, "copy_segments: row size %lld is not a multiple of 16 bytes",
                (long long) row_bytes);
    if (nseg == 0) return 0;
    PTB_REQUIRE(src_base && dst_bases && segments, PTB_ERR_ARG, "copy_segments: null pointer");
    PTB_REQUIRE(aligned16(src_base), PTB_ERR_ALIGN, "copy_segments: source is not 16-byte aligned");
    CopyArgs a{};
    a.src = (const uint8_t *) src_base;
    for (int r = 0; r < n_ranks; ++r) {
        PTB_REQUIRE(dst_bases[r] && aligned16(dst_bases[r]), PTB_ERR_ALIGN,
                    "copy_segments: destination of rank %d is null or not 16-byte aligned", r);
        a.dst[r] = (uint8_t *) dst_bases[r];
    }
    a.segs = segments; a.nseg = (int) nseg; a.n_ranks = n_ranks; a.row_bytes = row_bytes;
    int dev = 0, sms = 0;
    PTB_CUDA(cudaGetDevice(&dev));
    PTB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int grid = (num_ctas > 0) ? num_ctas : sms;
    copy_segments_kernel<<<grid, kCopyThreads, 0, (cudaStream_t) stream>>>(a);
    PTB_LAUNCH_CHECK("copy_segments_kernel");
    return 0;
}

int ptb_copy_segments_status(int *status, int reset) {
    PTB_REQUIRE(status, PTB_ERR_ARG, "copy_segments_status: null pointer");
    PTB_CUDA(cudaMemcpyFromSymbol(status, g_copy_error, sizeof(int)));
    if (reset) {
        int zero = 0;
        PTB_CUDA(cudaMemcpyToSymbol(g_copy_error, &zero, sizeof(int)));
    }
    return 0;
}

int ptb_gather_rows(const void *in, const int64_t *index, int64_t n_out, int64_t n_in, int64_t row_bytes, void *out,
                    ptb_stream_t stream) {
    PTB_REQUIRE(n_out >= 0 && n_in >= 0, PTB_ERR_ARG, "gather_rows: negative size");
    PTB_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0, PTB_ERR_ALIGN, "gather_rows: row size %lld is not a multiple of 16 bytes",
                (long long) row_bytes);
    if (n_out == 0) return 0;
    PTB_REQUIRE(index && out && (n_in == 0 || in), PTB_ERR_ARG, "gather_rows: null pointer");
    PTB_REQUIRE(aligned16(out) && (n_in == 0 || aligned16(in)), PTB_ERR_ALIGN, "gather_rows: buffers must be 16-byte aligned");
    const int64_t warps = n_out;
    const int blocks    = (int) imin(cdiv<int64_t>(warps, 8), 148 * 16);
    gather_rows_kernel<<<blocks, 256, 0, (cudaStream_t) stream>>>((const uint8_t *) in, index, n_out, n_in, row_bytes,
                                                                   (uint8_t *) out);
    PTB_LAUNCH_CHECK("gather_rows_kernel");
    return 0;
}

#pragma GCC visibility pop
} // extern "C"
