// Row-segment copies between GPUs of one node (the expert-parallel dispatch and combine), and the
// MoE row permutation kernels that sit either side of the grouped GEMM.
//
// Dispatch and combine are the same operation: every rank holds rows that are contiguous per
// (destination rank, expert) and knows, from the routing counts of all ranks, the row at which each
// such segment starts in the destination's buffer.  One kernel copies all segments of a rank with plain
// 16-byte loads from local memory and plain 16-byte stores to the destination -- peer memory mapped
// into this process (NVLink / NVSwitch) or local memory for the rank's own share -- so rows land in
// expert-major order, ready for the grouped GEMM, with no staging pass on either side.  The copy kernel
// waits on nothing.  Ordering between ranks: either a collective afterwards, or the copy's own signal --
// the last CTA to finish stores the exchange's sequence number into a slot of every destination's flag
// array (release, system scope, after every thread has fenced its data stores), and the destination runs
// a one-warp kernel that waits, with a time limit, until all sources' slots carry that number.
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
    // optional arrival signal (done == nullptr: none)
    uint32_t *flag[kMaxPeers]; // per destination rank: this rank's slot in that rank's flag array
    uint32_t *done;            // local counter of finished CTAs, zero between launches
    uint32_t seq;
};

constexpr uint64_t kFlagWaitLimitNs = 20000000000ull; // 20 s: ranks of one job are never this far apart

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// set to 1 by a copy whose segment table names a rank outside [0, n_ranks) (that segment is skipped),
// to 2 by a flag wait that ran out of time
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
    if (a.done != nullptr) {
        __threadfence_system(); // this thread's stores, wherever they went, before the CTA counts itself
        __syncthreads();
        if (tid == 0) {
            __threadfence_system();
            if (atomicAdd(a.done, 1u) == gridDim.x - 1) {
                __threadfence_system();
                for (int r = 0; r < a.n_ranks; ++r) st_release_sys(a.flag[r], a.seq);
                *a.done = 0; // the next launch on this stream starts after this kernel has ended
            }
        }
    }
}

// One warp: lane r waits until flags[r] has reached `seq` (sequence numbers only grow; the comparison
// survives wrap-around).  On expiry it records the failure and returns -- the stream goes on with
// whatever arrived, and the host finds the status word set.
__global__ void __launch_bounds__(32) wait_flags_kernel(const uint32_t *flags, int n, uint32_t seq) {
    const int r = threadIdx.x;
    if (r >= n) return;
    uint64_t t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    while ((int32_t) (ld_acquire_sys(flags + r) - seq) < 0) {
        __nanosleep(100);
        uint64_t t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        if (t - t0 > kFlagWaitLimitNs) {
            atomicExch(&g_copy_error, 2);
            break;
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

// ---- MoE token permutation: routing map -> expert-major positions --------------------------------------
// routing_map [T, E] (one byte per entry, non-zero = token t goes to expert e).  Position of (t, e) in
// the permuted order = rows of experts below e + tokens below t routed to e: a stable counting sort in
// three passes over blocks of kTokBlock tokens (count per block and expert, scan, assign).
constexpr int kTokBlock = 256;

__global__ void __launch_bounds__(256) moe_count_kernel(const uint8_t *__restrict__ map, int64_t T, int64_t E,
                                                         int *__restrict__ block_counts) {
    const int64_t t0 = (int64_t) blockIdx.x * kTokBlock, t1 = imin(t0 + kTokBlock, T);
    for (int64_t e = threadIdx.x; e < E; e += blockDim.x) {
        int c = 0;
        for (int64_t t = t0; t < t1; ++t) c += map[t * E + e] != 0;
        block_counts[(int64_t) blockIdx.x * E + e] = c;
    }
}

// one CTA: per expert, exclusive scan of the block counts over the token blocks; then the experts' first
// positions (exclusive scan over experts, done by thread 0: E is at most a few thousand)
__global__ void __launch_bounds__(256) moe_scan_kernel(int *__restrict__ block_counts, int64_t B, int64_t E,
                                                        int64_t *__restrict__ tokens_per_expert,
                                                        int64_t *__restrict__ expert_start) {
    for (int64_t e = threadIdx.x; e < E; e += blockDim.x) {
        int run = 0;
        for (int64_t b = 0; b < B; ++b) {
            const int c              = block_counts[b * E + e];
            block_counts[b * E + e] = run;
            run += c;
        }
        tokens_per_expert[e] = run;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int64_t run = 0;
        for (int64_t e = 0; e < E; ++e) {
            expert_start[e] = run;
            run += tokens_per_expert[e];
        }
        expert_start[E] = run;
    }
}

__global__ void __launch_bounds__(256) moe_assign_kernel(const uint8_t *__restrict__ map, int64_t T, int64_t E,
                                                          const int *__restrict__ block_counts,
                                                          const int64_t *__restrict__ expert_start, int64_t capacity,
                                                          int *__restrict__ row_id_map,
                                                          int64_t *__restrict__ sorted_indices) {
    const int64_t t0 = (int64_t) blockIdx.x * kTokBlock, t1 = imin(t0 + kTokBlock, T);
    for (int64_t e = threadIdx.x; e < E; e += blockDim.x) {
        int64_t pos = expert_start[e] + block_counts[(int64_t) blockIdx.x * E + e];
        for (int64_t t = t0; t < t1; ++t) {
            int id = -1;
            if (map[t * E + e] != 0) {
                if (pos < capacity) {
                    id = (int) pos;
                    if (sorted_indices != nullptr) sorted_indices[pos] = t;
                }
                ++pos;
            }
            row_id_map[t * E + e] = id;
        }
    }
}

// ---- weighted row gather: out[i] = cast(float(in[index[i]]) * w[i]) ---------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) gather_rows_scaled_kernel(const T *__restrict__ in, const int64_t *__restrict__ index,
                                                                  const float *__restrict__ weights, int64_t n_out,
                                                                  int64_t n_in, int64_t H, T *__restrict__ out) {
    const int lane   = threadIdx.x & 31;
    const int64_t w  = ((int64_t) blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nw = ((int64_t) gridDim.x * blockDim.x) >> 5;
    for (int64_t r = w; r < n_out; r += nw) {
        const int64_t s = index[r];
        const float wt  = weights[r];
        const bool ok   = s >= 0 && s < n_in;
        for (int64_t j = lane; j < H; j += 32)
            out[r * H + j] = from_f32<T>(ok ? __fmul_rn(to_f32(in[s * H + j]), wt) : 0.0f);
    }
}

// ---- un-permute: out[t] = sum over the experts e of token t, in increasing e, of in[pos(t,e)] * p(t,e) ------
// One warp per token.  The (at most E) positions of the token are compacted into shared memory first,
// then every lane walks its columns once per position.  Products and sums are separate fp32 operations
// (no contraction), accumulated in expert order: the result equals a sequential fp32 scatter-add.
constexpr int kUnpermWarps = 4;
constexpr int kMaxExperts  = 1024;

template <typename T, bool WITH_GRAD>
__global__ void __launch_bounds__(kUnpermWarps * 32) unpermute_kernel(
    const T *__restrict__ in, const int *__restrict__ row_id_map, const float *__restrict__ probs, int64_t T_, int64_t E,
    int64_t H, T *__restrict__ out,
    // WITH_GRAD: `in` is the gradient of the un-permuted rows [T, H], `fwd_in` the permuted rows of the
    // forward pass; writes grad_in[pos] = g[t] * p and grad_probs[t, e] = dot(g[t], fwd_in[pos])
    const T *__restrict__ fwd_in, float *__restrict__ grad_probs) {
    __shared__ int s_pos[kUnpermWarps][kMaxExperts];
    __shared__ int s_exp[kUnpermWarps][kMaxExperts];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t t = (int64_t) blockIdx.x * kUnpermWarps + warp;
    if (t >= T_) return;
    int n = 0;
    for (int64_t base = 0; base < E; base += 32) {
        const int64_t e = base + lane;
        const int id    = e < E ? row_id_map[t * E + e] : -1;
        const unsigned m = __ballot_sync(0xffffffffu, id >= 0);
        if (id >= 0) {
            const int k  = n + __popc(m & ((1u << lane) - 1));
            s_pos[warp][k] = id;
            s_exp[warp][k] = (int) e;
        }
        if (WITH_GRAD && grad_probs != nullptr && e < E && id < 0) grad_probs[t * E + e] = 0.0f;
        n += __popc(m);
    }
    __syncwarp();
    if constexpr (!WITH_GRAD) {
        for (int64_t j = lane; j < H; j += 32) {
            float acc = 0.0f;
            for (int k = 0; k < n; ++k) {
                float v = to_f32(in[(int64_t) s_pos[warp][k] * H + j]);
                if (probs != nullptr) v = __fmul_rn(v, probs[t * E + s_exp[warp][k]]);
                acc = __fadd_rn(acc, v);
            }
            out[t * H + j] = from_f32<T>(acc);
        }
    } else {
        for (int k = 0; k < n; ++k) {
            const int64_t pos = s_pos[warp][k];
            const float p     = probs != nullptr ? probs[t * E + s_exp[warp][k]] : 1.0f;
            float dot         = 0.0f;
            for (int64_t j = lane; j < H; j += 32) {
                const float g = to_f32(in[t * H + j]);
                out[pos * H + j] = from_f32<T>(__fmul_rn(g, p));
                if (grad_probs != nullptr) dot += g * to_f32(fwd_in[pos * H + j]);
            }
            if (grad_probs != nullptr) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                if (lane == 0) grad_probs[t * E + s_exp[warp][k]] = dot;
            }
        }
    }
}

} // namespace
} // namespace ptb

using namespace ptb;

extern "C" {
#pragma GCC visibility push(default)

static int copy_segments_impl(const void *src_base, void *const *dst_bases, int n_ranks, const int64_t *segments,
                              int64_t nseg, int64_t row_bytes, int num_ctas, void *const *flag_slots, void *done_counter,
                              uint32_t seq, ptb_stream_t stream);

int ptb_copy_segments(const void *src_base, void *const *dst_bases, int n_ranks, const int64_t *segments, int64_t nseg,
                      int64_t row_bytes, int num_ctas, ptb_stream_t stream) {
    return copy_segments_impl(src_base, dst_bases, n_ranks, segments, nseg, row_bytes, num_ctas, nullptr, nullptr, 0, stream);
}

int ptb_copy_segments_signal(const void *src_base, void *const *dst_bases, int n_ranks, const int64_t *segments,
                             int64_t nseg, int64_t row_bytes, int num_ctas, void *const *flag_slots, void *done_counter,
                             uint32_t seq, ptb_stream_t stream) {
    PTB_REQUIRE(flag_slots && done_counter, PTB_ERR_ARG, "copy_segments_signal: null flag slots or counter");
    return copy_segments_impl(src_base, dst_bases, n_ranks, segments, nseg, row_bytes, num_ctas, flag_slots, done_counter, seq,
                              stream);
}

int ptb_wait_flags(const void *flags, int n, uint32_t seq, ptb_stream_t stream) {
    PTB_REQUIRE(flags && n >= 1 && n <= 32, PTB_ERR_ARG, "wait_flags: 1 to 32 flags");
    wait_flags_kernel<<<1, 32, 0, (cudaStream_t) stream>>>((const uint32_t *) flags, n, seq);
    PTB_LAUNCH_CHECK("wait_flags_kernel");
    return 0;
}

static int copy_segments_impl(const void *src_base, void *const *dst_bases, int n_ranks, const int64_t *segments,
                              int64_t nseg, int64_t row_bytes, int num_ctas, void *const *flag_slots, void *done_counter,
                              uint32_t seq, ptb_stream_t stream) {
    PTB_REQUIRE(n_ranks >= 1 && n_ranks <= kMaxPeers, PTB_ERR_TOO_LARGE, "copy_segments: 1 to %d ranks, got %d", kMaxPeers,
                n_ranks);
    PTB_REQUIRE(nseg >= 0 && nseg <= kMaxSegments, PTB_ERR_TOO_LARGE, "copy_segments: at most %d segments", kMaxSegments);
    PTB_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0, PTB_ERR_ALIGN, "copy_segments: row size %lld is not a multiple of 16 bytes",
                (long long) row_bytes);
    if (nseg == 0 && flag_slots == nullptr) return 0;
    PTB_REQUIRE(dst_bases && (nseg == 0 || (src_base && segments)), PTB_ERR_ARG, "copy_segments: null pointer");
    PTB_REQUIRE(aligned16(src_base), PTB_ERR_ALIGN, "copy_segments: source is not 16-byte aligned");
    CopyArgs a{};
    a.src = (const uint8_t *) src_base;
    for (int r = 0; r < n_ranks; ++r) {
        PTB_REQUIRE(dst_bases[r] && aligned16(dst_bases[r]), PTB_ERR_ALIGN,
                    "copy_segments: destination of rank %d is null or not 16-byte aligned", r);
        a.dst[r] = (uint8_t *) dst_bases[r];
    }
    a.segs = segments; a.nseg = (int) nseg; a.n_ranks = n_ranks; a.row_bytes = row_bytes;
    if (flag_slots != nullptr) {
        for (int r = 0; r < n_ranks; ++r) {
            PTB_REQUIRE(flag_slots[r] && (reinterpret_cast<uintptr_t>(flag_slots[r]) & 3u) == 0, PTB_ERR_ALIGN,
                        "copy_segments_signal: flag slot of rank %d is null or misaligned", r);
            a.flag[r] = (uint32_t *) flag_slots[r];
        }
        a.done = (uint32_t *) done_counter;
        a.seq  = seq;
    }
    int dev = 0, sms = 0;
    PTB_CUDA(cudaGetDevice(&dev));
    PTB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int grid = (num_ctas > 0) ? num_ctas : sms;
    copy_segments_kernel<<<grid, kCopyThreads, 0, (cudaStream_t) stream>>>(a);
    PTB_LAUNCH_CHECK("copy_segments_kernel");
    return 0;
}

int ptb_enable_peer_access(int peer_device) {
    int dev = -1;
    PTB_CUDA(cudaGetDevice(&dev));
    if (peer_device == dev) return 0;
    int can = 0;
    PTB_CUDA(cudaDeviceCanAccessPeer(&can, dev, peer_device));
    PTB_REQUIRE(can, PTB_ERR_UNSUPPORTED, "device %d cannot address the memory of device %d", dev, peer_device);
    const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        (void) cudaGetLastError(); // not an error: clear it
        return 0;
    }
    if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceEnablePeerAccess");
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

int ptb_moe_row_id_map(const void *routing_map, int64_t T, int64_t E, int64_t capacity, int32_t *row_id_map,
                       int64_t *tokens_per_expert, int64_t *sorted_indices, void *workspace, ptb_stream_t stream) {
    PTB_REQUIRE(T >= 0 && E >= 0 && capacity >= 0, PTB_ERR_ARG, "moe_row_id_map: negative size");
    PTB_REQUIRE(E <= kMaxExperts, PTB_ERR_TOO_LARGE, "moe_row_id_map: at most %d experts", kMaxExperts);
    PTB_REQUIRE(T * E < 2147483647LL && capacity < 2147483647LL, PTB_ERR_TOO_LARGE, "moe_row_id_map: problem too large");
    if (E == 0) return 0;
    PTB_REQUIRE(tokens_per_expert && workspace, PTB_ERR_ARG, "moe_row_id_map: null pointer");
    const int64_t B = cdiv<int64_t>(T, kTokBlock);
    int *block_counts     = (int *) workspace;                               // [B, E] int32
    int64_t *expert_start = (int64_t *) ((uint8_t *) workspace + ((B * E * 4 + 15) / 16) * 16); // [E + 1] int64
    cudaStream_t st = (cudaStream_t) stream;
    if (T > 0) {
        PTB_REQUIRE(routing_map && row_id_map, PTB_ERR_ARG, "moe_row_id_map: null pointer");
        moe_count_kernel<<<(unsigned) B, 256, 0, st>>>((const uint8_t *) routing_map, T, E, block_counts);
        PTB_LAUNCH_CHECK("moe_count_kernel");
    }
    moe_scan_kernel<<<1, 256, 0, st>>>(block_counts, B, E, tokens_per_expert, expert_start);
    PTB_LAUNCH_CHECK("moe_scan_kernel");
    if (T > 0) {
        moe_assign_kernel<<<(unsigned) B, 256, 0, st>>>((const uint8_t *) routing_map, T, E, block_counts, expert_start,
                                                         capacity, row_id_map, sorted_indices);
        PTB_LAUNCH_CHECK("moe_assign_kernel");
    }
    return 0;
}

int ptb_gather_rows_scaled(const void *in, int dtype, const int64_t *index, const float *weights, int64_t n_out,
                           int64_t n_in, int64_t H, void *out, ptb_stream_t stream) {
    PTB_REQUIRE(n_out >= 0 && n_in >= 0 && H >= 0, PTB_ERR_ARG, "gather_rows_scaled: negative size");
    if (n_out == 0 || H == 0) return 0;
    PTB_REQUIRE(index && weights && out && (n_in == 0 || in), PTB_ERR_ARG, "gather_rows_scaled: null pointer");
    const int blocks = (int) imin(cdiv<int64_t>(n_out, 8), 148 * 16);
    PTB_SWITCH_HP(dtype, T, (gather_rows_scaled_kernel<T><<<blocks, 256, 0, (cudaStream_t) stream>>>(
                                (const T *) in, index, weights, n_out, n_in, H, (T *) out)));
    PTB_LAUNCH_CHECK("gather_rows_scaled_kernel");
    return 0;
}

int ptb_unpermute_rows(const void *in, int dtype, const int32_t *row_id_map, const float *probs, int64_t T, int64_t E,
                       int64_t H, void *out, ptb_stream_t stream) {
    PTB_REQUIRE(T >= 0 && E >= 0 && H >= 0, PTB_ERR_ARG, "unpermute_rows: negative size");
    PTB_REQUIRE(E <= kMaxExperts, PTB_ERR_TOO_LARGE, "unpermute_rows: at most %d experts", kMaxExperts);
    if (T == 0 || H == 0) return 0;
    PTB_REQUIRE(out && row_id_map, PTB_ERR_ARG, "unpermute_rows: null pointer");
    const unsigned grid = (unsigned) cdiv<int64_t>(T, kUnpermWarps);
    PTB_SWITCH_HP(dtype, TT, (unpermute_kernel<TT, false><<<grid, kUnpermWarps * 32, 0, (cudaStream_t) stream>>>(
                                 (const TT *) in, row_id_map, probs, T, E, H, (TT *) out, nullptr, nullptr)));
    PTB_LAUNCH_CHECK("unpermute_kernel");
    return 0;
}

int ptb_unpermute_rows_bwd(const void *grad_out, int dtype, const void *fwd_in, const int32_t *row_id_map,
                           const float *probs, int64_t T, int64_t E, int64_t H, void *grad_in, float *grad_probs,
                           ptb_stream_t stream) {
    PTB_REQUIRE(T >= 0 && E >= 0 && H >= 0, PTB_ERR_ARG, "unpermute_rows_bwd: negative size");
    PTB_REQUIRE(E <= kMaxExperts, PTB_ERR_TOO_LARGE, "unpermute_rows_bwd: at most %d experts", kMaxExperts);
    if (T == 0 || H == 0) return 0;
    PTB_REQUIRE(grad_out && grad_in && row_id_map, PTB_ERR_ARG, "unpermute_rows_bwd: null pointer");
    PTB_REQUIRE(grad_probs == nullptr || fwd_in != nullptr, PTB_ERR_ARG, "unpermute_rows_bwd: grad_probs needs the forward rows");
    const unsigned grid = (unsigned) cdiv<int64_t>(T, kUnpermWarps);
    PTB_SWITCH_HP(dtype, TT, (unpermute_kernel<TT, true><<<grid, kUnpermWarps * 32, 0, (cudaStream_t) stream>>>(
                                 (const TT *) grad_out, row_id_map, probs, T, E, H, (TT *) grad_in, (const TT *) fwd_in,
                                 grad_probs)));
    PTB_LAUNCH_CHECK("unpermute_kernel");
    return 0;
}

#pragma GCC visibility pop
} // extern "C"
