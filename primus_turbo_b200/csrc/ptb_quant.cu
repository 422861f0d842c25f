// FP8 quantize / dequantize kernels and their C entry points (sm_100a).
//
// All of these are HBM-bandwidth bound: every kernel reads its input once with 16-byte loads
// (twice for the two-pass tensorwise / rowwise reductions, whose second pass is served largely
// from the 126 MB L2), keeps the tile in registers, reduces the amax with warp shuffles and
// shared memory, and writes FP8 with 8-byte stores.
#include <atomic>

#include "ptb_common.cuh"

namespace ptb {

thread_local char g_err[kErrBufLen] = {0};
char *err_buf() { return g_err; }

namespace {

constexpr float kEpsTensorRow = 1e-12f; // tensorwise / rowwise floor of the amax
constexpr float kEpsBlock     = 1e-4f;  // blockwise floor of the amax
constexpr int kBlk            = 128;    // block size of the blockwise granularities

// ---- 8-element row fragment load / store -----------------------------------------------------
template <typename T>
__device__ __forceinline__ void load8(const T *__restrict__ row, int64_t col, int64_t ncols, bool vec,
                                      float (&v)[8]) {
    if (vec && col + 8 <= ncols) {
        if constexpr (sizeof(T) == 2) {
            uint4 raw = *reinterpret_cast<const uint4 *>(row + col);
            const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = to_f32(e[i]);
        } else {
            float4 a = *reinterpret_cast<const float4 *>(row + col);
            float4 b = *reinterpret_cast<const float4 *>(row + col + 4);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
            v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = (col + i < ncols) ? to_f32(row[col + i]) : 0.0f;
    }
}

template <int FMT>
__device__ __forceinline__ void store8_fp8(uint8_t *__restrict__ row, int64_t col, int64_t ncols, bool vec,
                                           const float (&v)[8]) {
    uint16_t p0 = cvt_fp8x2<FMT>(v[0], v[1]);
    uint16_t p1 = cvt_fp8x2<FMT>(v[2], v[3]);
    uint16_t p2 = cvt_fp8x2<FMT>(v[4], v[5]);
    uint16_t p3 = cvt_fp8x2<FMT>(v[6], v[7]);
    if (vec && col + 8 <= ncols) {
        uint2 out;
        out.x = (uint32_t) p0 | ((uint32_t) p1 << 16);
        out.y = (uint32_t) p2 | ((uint32_t) p3 << 16);
        *reinterpret_cast<uint2 *>(row + col) = out;
    } else {
        uint16_t p[4] = {p0, p1, p2, p3};
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (col + i < ncols) row[col + i] = (uint8_t) ((p[i >> 1] >> ((i & 1) * 8)) & 0xff);
    }
}

// ---- 128x128 tile quantize: row blocks, column blocks, whole tile, segment-padded ------------
constexpr int kModeRow = 1; // 1x128 scales
constexpr int kModeCol = 2; // 128x1 scales
constexpr int kMode2D  = 4; // one scale per tile

struct BlockQuantArgs {
    const void *x;
    uint8_t *q_row;   // row-scaled copy (or the only copy in 2-D mode)
    uint8_t *q_col;   // column-scaled copy
    float *s_row;     // [.. m*s_row_stride_m + nb*s_row_stride_nb]
    float *s_col;     // [mb, N]
    float *s_2d;      // [b, mb, nb]
    int64_t B, M, N;
    int64_t s_row_stride_m, s_row_stride_nb;
    // segment mode
    int64_t G;
    const int64_t *group_offs;
    const int64_t *var_k_offs; // padded offsets, written by segment_offsets_kernel before the tile kernel runs
    const int2 *block_table;   // optional: per padded 128-row block {first source row, end of its group's rows}
    // fused activation (ACT = 1): x is [M, 2N] (gate half, then linear half), the tile that is quantised is
    // swiglu_prob(x[:, :N], x[:, N:], act_probs[row]) rounded to the input type first
    const float *act_probs;
    int64_t x_ld; // row pitch of x in elements (N, or 2N with the fused activation)
};

// 8 consecutive elements of the tile's source row `r`, columns col .. col+7 (all in range), as stored bits
template <typename T, int ACT>
__device__ __forceinline__ uint4 load_tile8(const T *__restrict__ xrow, int64_t col, int64_t N, float prob) {
    if constexpr (ACT == 0) {
        return *reinterpret_cast<const uint4 *>(xrow + col);
    } else {
        const uint4 u = *reinterpret_cast<const uint4 *>(xrow + col);
        const uint4 d = *reinterpret_cast<const uint4 *>(xrow + N + col);
        const T *ue = reinterpret_cast<const T *>(&u), *de = reinterpret_cast<const T *>(&d);
        uint4 o;
        T *oe = reinterpret_cast<T *>(&o);
#pragma unroll
        for (int i = 0; i < 8; ++i) oe[i] = from_f32<T>(swiglu_prob(to_f32(ue[i]), to_f32(de[i]), prob));
        return o;
    }
}

template <typename T> struct Packed2;
template <> struct Packed2<__nv_bfloat16> {
    using type = __nv_bfloat162;
    static __device__ __forceinline__ type zero() { return __floats2bfloat162_rn(0.f, 0.f); }
    static __device__ __forceinline__ float2 to_float2(type v) { return __bfloat1622float2(v); }
};
template <> struct Packed2<__half> {
    using type = __half2;
    static __device__ __forceinline__ type zero() { return __floats2half2_rn(0.f, 0.f); }
    static __device__ __forceinline__ float2 to_float2(type v) { return __half22float2(v); }
};
template <> struct Packed2<float> {
    using type = float2;
    static __device__ __forceinline__ type zero() { return make_float2(0.f, 0.f); }
};

template <int FMT, typename T> __device__ __forceinline__ void scale_store8_t(const uint4 &raw, const float2 (&s)[4], uint8_t *dst) {
    using T2    = typename Packed2<T>::type;
    const T2 *e = reinterpret_cast<const T2 *>(&raw);
    uint32_t o[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const float2 lo = __fmul2_rn(Packed2<T>::to_float2(e[2 * h]), s[2 * h]);
        const float2 hi = __fmul2_rn(Packed2<T>::to_float2(e[2 * h + 1]), s[2 * h + 1]);
        o[h] = (uint32_t) cvt_fp8x2<FMT>(lo.x, lo.y) | ((uint32_t) cvt_fp8x2<FMT>(hi.x, hi.y) << 16);
    }
    *reinterpret_cast<uint2 *>(dst) = make_uint2(o[0], o[1]);
}

// One 8-element row fragment kept in its storage format: 16 bytes for 16-bit inputs, so a thread's
// 8x8 share of the tile costs 32 registers and is decoded on the fly in each pass.
template <typename T> struct RowFrag {
    uint4 raw;
    __device__ __forceinline__ void zero() { raw = make_uint4(0, 0, 0, 0); }
    __device__ __forceinline__ void load(const T *row, int64_t col, int64_t ncols, bool vec) {
        if (vec && col + 8 <= ncols) {
            raw = *reinterpret_cast<const uint4 *>(row + col);
        } else {
            T e[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) e[i] = (col + i < ncols) ? row[col + i] : from_f32<T>(0.0f);
            raw = *reinterpret_cast<const uint4 *>(e);
        }
    }
    __device__ __forceinline__ void decode(float (&v)[8]) const {
        const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = to_f32(e[i]);
    }
};
template <> struct RowFrag<float> {
    float4 lo, hi;
    __device__ __forceinline__ void zero() { lo = hi = make_float4(0.f, 0.f, 0.f, 0.f); }
    __device__ __forceinline__ void load(const float *row, int64_t col, int64_t ncols, bool vec) {
        float v[8];
        load8<float>(row, col, ncols, vec, v);
        lo = make_float4(v[0], v[1], v[2], v[3]);
        hi = make_float4(v[4], v[5], v[6], v[7]);
    }
    __device__ __forceinline__ void decode(float (&v)[8]) const {
        v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w;
        v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
    }
};

// var_k_lens[g] = ceil(len_g / 128) * 128 and its exclusive prefix var_k_offs[G+1] (one CTA).  With a
// block table, also: for every 128-row block of the padded layout, the first source row it holds and
// the end of its group's source rows -- so the tile kernel finds its rows with one load instead of
// scanning the offsets of all groups.
__global__ void __launch_bounds__(256) segment_offsets_kernel(const int64_t *__restrict__ group_offs, int64_t G,
                                                               int64_t *__restrict__ var_k_lens,
                                                               int64_t *__restrict__ var_k_offs,
                                                               int2 *__restrict__ block_table) {
    __shared__ int64_t s_scan[256];
    const int tid     = threadIdx.x;
    const int64_t per = cdiv<int64_t>(G, 256);
    const int64_t g0 = (int64_t) tid * per, g1 = imin(g0 + per, G);
    int64_t local = 0;
    for (int64_t g = g0; g < g1; ++g) local += cdiv<int64_t>(group_offs[g + 1] - group_offs[g], kBlk) * kBlk;
    s_scan[tid] = local;
    __syncthreads();
    for (int off = 1; off < 256; off <<= 1) {
        int64_t add = (tid >= off) ? s_scan[tid - off] : 0;
        __syncthreads();
        s_scan[tid] += add;
        __syncthreads();
    }
    int64_t run = s_scan[tid] - local;
    for (int64_t g = g0; g < g1; ++g) {
        const int64_t gs = group_offs[g], ge = group_offs[g + 1];
        const int64_t pl = cdiv<int64_t>(ge - gs, kBlk) * kBlk;
        var_k_lens[g]    = pl;
        var_k_offs[g]    = run;
        if (block_table != nullptr) {
            for (int64_t t = 0; t < pl / kBlk; ++t)
                block_table[run / kBlk + t] = make_int2((int) (gs + t * kBlk), (int) ge);
        }
        run += pl;
    }
    if (tid == 255) var_k_offs[G] = s_scan[255];
}

// Segment row + column quantiser for 16-bit inputs whose width is a multiple of 128 (the MoE activation and
// grad-out shapes), with the block table.  One CTA walks kSegStrip consecutive column tiles of one padded
// 128-row block.  The tile after the one being processed is already on its way: every thread copies its
// own eight 16-byte fragments with cp.async into eight private shared-memory slots (rows past the group's
// end are zero-filled by the copy itself), reads them back into registers when the tile's turn comes and
// at once issues the copies of the following tile into the same slots -- so global loads are in flight
// during all of the arithmetic and the stores, and ragged tiles run the same code as full ones (only the
// row-direction stores are predicated).  Arithmetic and results are those of quant_block_kernel.
// Build-time switches for A/B measurements: the streamed kernel on / off, and the column tiles one CTA walks
// (activation 65536 x 7168 bf16, 256 groups: general tile kernel 0.47 ms, strips of 2 / 4 / 8 tiles
// 0.40 / 0.42 / 0.53 ms).
#ifndef PTB_SEG_STREAM
#define PTB_SEG_STREAM 1
#endif
#ifndef PTB_SEG_STRIP
#define PTB_SEG_STRIP 2
#endif
constexpr int kSegStrip = PTB_SEG_STRIP;

__device__ __forceinline__ void cp_async16_zfill(void *dst_smem, const void *src, bool valid) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t) __cvta_generic_to_shared(dst_smem)), "l"(src),
                 "r"(valid ? 16u : 0u)
                 : "memory");
}

template <typename T, int FMT>
__global__ void __launch_bounds__(256, 3) seg_quant_stream_kernel(const BlockQuantArgs p) {
    __shared__ uint4 s_frag[8][256];
    __shared__ float s_colmax[16][kBlk + 1];
    __shared__ float s_colscale[kBlk];
    using T2 = typename Packed2<T>::type;

    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const uint32_t tiles_n = (uint32_t) (p.N / kBlk);
    const uint32_t strips  = (tiles_n + kSegStrip - 1) / kSegStrip;
    const uint32_t tm      = blockIdx.x / strips;
    const uint32_t tn0     = (blockIdx.x - tm * strips) * kSegStrip;
    const int ntiles       = (int) min((uint32_t) kSegStrip, tiles_n - tn0);
    if ((int64_t) tm * kBlk >= p.var_k_offs[p.G]) return; // block lies beyond the last padded segment
    const int2 e          = p.block_table[tm];
    const int64_t in_row0 = e.x, in_end = e.y, out_row0 = (int64_t) tm * kBlk;
    const T *xb           = reinterpret_cast<const T *>(p.x);
    // source pointers of this thread's eight fragments in the strip's first tile (clamped rows are never read)
    bool valid[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) valid[i] = in_row0 + ty + 16 * i < in_end;
    const T *src0 = xb + (in_row0 + ty) * p.N + (int64_t) tn0 * kBlk + tx * 8;
    const int64_t step = 16 * p.N;

    auto issue = [&](int t) {
#pragma unroll
        for (int i = 0; i < 8; ++i) cp_async16_zfill(&s_frag[i][tid], valid[i] ? src0 + i * step + t * kBlk : xb, valid[i]);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    issue(0);
    for (int t = 0; t < ntiles; ++t) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        uint4 raw[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) raw[i] = s_frag[i][tid];
        if (t + 1 < ntiles) issue(t + 1); // own slots only: no other thread reads or writes them
        const int64_t tn  = tn0 + t;
        const int64_t col = tn * kBlk + tx * 8;

        T2 cm2[4];
        float rm[8];
#pragma unroll
        for (int w = 0; w < 4; ++w) cm2[w] = Packed2<T>::zero();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const T2 *el = reinterpret_cast<const T2 *>(&raw[i]);
            T2 a[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                a[w]   = __habs2(el[w]);
                cm2[w] = __hmax2(cm2[w], a[w]);
            }
            const T2 m2 = __hmax2(__hmax2(a[0], a[1]), __hmax2(a[2], a[3]));
            rm[i]       = fmaxf(to_f32(m2.x), to_f32(m2.y));
        }
        // ---- row direction: 16 lanes share a row; one lane per row does the two divisions -------------
#pragma unroll
        for (int i = 0; i < 8; ++i) {
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) rm[i] = fmaxf(rm[i], __shfl_xor_sync(0xffffffffu, rm[i], o));
        }
        float mine = rm[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) mine = ((tx & 7) == i) ? rm[i] : mine;
        float sc_mine, sci_mine;
        scale_from_amax<FMT>(mine, kEpsBlock, sc_mine, sci_mine);
        if (tx < 8 && in_row0 + ty + 16 * tx < in_end)
            p.s_row[(in_row0 + ty + 16 * tx) * p.s_row_stride_m + tn * p.s_row_stride_nb] = sci_mine;
        const int half_base = (tid & 31) & 16;
        uint8_t *dst_row    = p.q_row + (in_row0 + ty) * p.N + col;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float sc     = __shfl_sync(0xffffffffu, sc_mine, half_base + i);
            const float2 s2[4] = {make_float2(sc, sc), make_float2(sc, sc), make_float2(sc, sc), make_float2(sc, sc)};
            if (valid[i]) scale_store8_t<FMT, T>(raw[i], s2, dst_row + i * step);
        }
        // ---- column direction: the 16 row lanes meet in shared memory ------------------------------------
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            s_colmax[ty][tx * 8 + 2 * w]     = to_f32(cm2[w].x);
            s_colmax[ty][tx * 8 + 2 * w + 1] = to_f32(cm2[w].y);
        }
        __syncthreads();
        if (tid < kBlk) {
            float m = 0.0f;
#pragma unroll
            for (int k = 0; k < 16; ++k) m = fmaxf(m, s_colmax[k][tid]);
            float sc, sci;
            scale_from_amax<FMT>(m, kEpsBlock, sc, sci);
            s_colscale[tid]                         = sc;
            p.s_col[tm * p.N + tn * kBlk + tid] = sci;
        }
        __syncthreads();
        float2 s2[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) s2[w] = make_float2(s_colscale[tx * 8 + 2 * w], s_colscale[tx * 8 + 2 * w + 1]);
        uint8_t *dst_col = p.q_col + (out_row0 + ty) * p.N + col;
#pragma unroll
        for (int i = 0; i < 8; ++i) scale_store8_t<FMT, T>(raw[i], s2, dst_col + i * step);
        // the next tile's column maxima must not land before every thread has read this tile's scales
        __syncthreads();
    }
}

// Grid: one CTA per 128x128 tile, column tiles fastest, so that CTAs resident together stream whole
// contiguous row bands (DRAM pages are used end to end instead of 256 bytes at a time).
template <typename T, int FMT, int MODE, bool SEGMENT, int ACT = 0>
__global__ void __launch_bounds__(256, 3) quant_block_kernel(const BlockQuantArgs p) {
    __shared__ float s_colmax[16][kBlk + 1];
    __shared__ float s_colscale[kBlk];
    __shared__ float s_red[8];
    __shared__ int64_t s_seg[3]; // found, first source row, end of the group's source rows

    const int tid = threadIdx.x;
    const int tx  = tid & 15;  // 8-column fragment index inside the tile
    const int ty  = tid >> 4;  // row lane 0..15
    // the grid is at most 2^31 - 1 tiles (checked by the launcher): 32-bit divisions, a 64-bit one
    // costs each thread ~80 instructions
    const uint32_t tiles_n32 = (uint32_t) cdiv<int64_t>(p.N, kBlk);
    const uint32_t tiles_m32 = (uint32_t) cdiv<int64_t>(SEGMENT ? (p.M + p.G * kBlk) : p.M, kBlk);
    const uint32_t tmb32     = blockIdx.x / tiles_n32;
    const int64_t tiles_n = tiles_n32, tiles_m = tiles_m32;
    const int64_t tn      = blockIdx.x - tmb32 * tiles_n32;
    const int64_t b       = SEGMENT ? 0 : tmb32 / tiles_m32;
    const int64_t tm      = SEGMENT ? tmb32 : tmb32 - (uint32_t) b * tiles_m32;

    int64_t in_row0  = tm * kBlk; // first source row of this tile
    int64_t in_end   = p.M;       // first invalid source row
    const int64_t out_row0 = tm * kBlk;

    if constexpr (SEGMENT) {
        // find the source rows of this padded tile
        const int64_t block_start = tm * kBlk;
        if (p.block_table != nullptr) {
            // one load from the table written by the offsets kernel; tiles beyond the last padded
            // segment have nothing to do
            if (block_start >= p.var_k_offs[p.G]) return;
            const int2 e = p.block_table[tm];
            in_row0 = e.x;
            in_end  = e.y;
        } else {
            // no table: scan the groups (all four offsets of a candidate group are fetched in one round of
            // independent loads, and a single barrier both publishes the hit and tells every thread
            // whether there was one)
            int found = 0;
            for (int64_t g = tid; g < p.G; g += 256) {
                const int64_t ps = p.var_k_offs[g], pe = p.var_k_offs[g + 1];
                const int64_t gs = p.group_offs[g], ge = p.group_offs[g + 1];
                if (block_start >= ps && block_start < pe) {
                    found    = 1;
                    s_seg[1] = gs + (block_start - ps);
                    s_seg[2] = ge;
                }
            }
            if (!__syncthreads_or(found)) return; // tile lies beyond the last padded segment
            in_row0 = s_seg[1];
            in_end  = s_seg[2];
        }
    }

    const T *xb        = reinterpret_cast<const T *>(p.x) + b * p.M * p.x_ld;
    const int64_t col  = tn * kBlk + tx * 8;
    const bool vec_in  = (p.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.x) & 15u) == 0);
    const bool vec_out = (p.N % 8 == 0);

    if constexpr (MODE == kMode2D && !SEGMENT && sizeof(T) == 2) {
        // Interior 128x128 tile of a 16-bit weight: no per-row predicates, one running packed |x|
        // maximum, packed fp32x2 scaling.  Same arithmetic as the general path below.
        if (vec_in && in_row0 + kBlk <= p.M && (tn + 1) * kBlk <= p.N) {
            using T2 = typename Packed2<T>::type;
            const T *src = xb + (in_row0 + ty) * p.N + col;
            uint4 raw[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) raw[i] = *reinterpret_cast<const uint4 *>(src + (int64_t) (16 * i) * p.N);
            T2 m2 = Packed2<T>::zero();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const T2 *e = reinterpret_cast<const T2 *>(&raw[i]);
#pragma unroll
                for (int w = 0; w < 4; ++w) m2 = __hmax2(m2, __habs2(e[w]));
            }
            float m = warp_max(fmaxf(to_f32(m2.x), to_f32(m2.y)));
            if ((tid & 31) == 0) s_red[tid >> 5] = m;
            __syncthreads();
            m = s_red[0];
#pragma unroll
            for (int k = 1; k < 8; ++k) m = fmaxf(m, s_red[k]);
            float sc, sci;
            scale_from_amax<FMT>(m, kEpsBlock, sc, sci);
            const float2 sc2 = make_float2(sc, sc);
            uint8_t *dst     = p.q_row + b * p.M * p.N + (in_row0 + ty) * p.N + col;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const T2 *e = reinterpret_cast<const T2 *>(&raw[i]);
                uint32_t o[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const float2 lo = __fmul2_rn(Packed2<T>::to_float2(e[2 * h]), sc2);
                    const float2 hi = __fmul2_rn(Packed2<T>::to_float2(e[2 * h + 1]), sc2);
                    o[h] = (uint32_t) cvt_fp8x2<FMT>(lo.x, lo.y) | ((uint32_t) cvt_fp8x2<FMT>(hi.x, hi.y) << 16);
                }
                *reinterpret_cast<uint2 *>(dst + (int64_t) (16 * i) * p.N) = make_uint2(o[0], o[1]);
            }
            if (tid == 0) p.s_2d[(b * tiles_m + tm) * tiles_n + tn] = sci;
            return;
        }
    }

    if constexpr (MODE != kMode2D && sizeof(T) == 2) {
        // Interior tile (all 128 source rows and columns exist, 16-byte aligned rows) of a 16-bit
        // input: the general path's per-row predicates and 64-bit index products are hoisted out.
        // Same arithmetic, same results.
        if (vec_in && in_row0 + kBlk <= in_end && (tn + 1) * kBlk <= p.N) {
            using T2 = typename Packed2<T>::type;
            const T *src       = xb + (in_row0 + ty) * p.x_ld;
            const int64_t step = 16 * p.N; // row step of the outputs (16 rows of N columns)
            uint4 raw[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float prob = 1.0f;
                if constexpr (ACT != 0) prob = p.act_probs[in_row0 + ty + 16 * i];
                raw[i] = load_tile8<T, ACT>(src + (int64_t) (16 * i) * p.x_ld, col, p.N, prob);
            }
            T2 cm2[4];
            float rm[8];
#pragma unroll
            for (int w = 0; w < 4; ++w) cm2[w] = Packed2<T>::zero();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const T2 *e = reinterpret_cast<const T2 *>(&raw[i]);
                T2 a[4];
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    a[w] = __habs2(e[w]);
                    if constexpr (MODE & kModeCol) cm2[w] = __hmax2(cm2[w], a[w]);
                }
                const T2 m2 = __hmax2(__hmax2(a[0], a[1]), __hmax2(a[2], a[3]));
                rm[i]       = fmaxf(to_f32(m2.x), to_f32(m2.y));
            }
            if constexpr (MODE & kModeRow) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
#pragma unroll
                    for (int o = 8; o > 0; o >>= 1) rm[i] = fmaxf(rm[i], __shfl_xor_sync(0xffffffffu, rm[i], o));
                }
                float mine = rm[0];
#pragma unroll
                for (int i = 1; i < 8; ++i) mine = ((tx & 7) == i) ? rm[i] : mine;
                float sc_mine, sci_mine;
                scale_from_amax<FMT>(mine, kEpsBlock, sc_mine, sci_mine);
                if (tx < 8) p.s_row[(in_row0 + ty + 16 * tx) * p.s_row_stride_m + tn * p.s_row_stride_nb] = sci_mine;
                const int half_base = (tid & 31) & 16;
                uint8_t *dst        = p.q_row + b * p.M * p.N + (in_row0 + ty) * p.N + col;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float sc = __shfl_sync(0xffffffffu, sc_mine, half_base + i);
                    const float2 s2[4] = {make_float2(sc, sc), make_float2(sc, sc), make_float2(sc, sc), make_float2(sc, sc)};
                    scale_store8_t<FMT, T>(raw[i], s2, dst + i * step);
                }
            }
            if constexpr (MODE & kModeCol) {
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    s_colmax[ty][tx * 8 + 2 * w]     = to_f32(cm2[w].x);
                    s_colmax[ty][tx * 8 + 2 * w + 1] = to_f32(cm2[w].y);
                }
                __syncthreads();
                if (tid < kBlk) {
                    float m = 0.0f;
#pragma unroll
                    for (int k = 0; k < 16; ++k) m = fmaxf(m, s_colmax[k][tid]);
                    float sc, sci;
                    scale_from_amax<FMT>(m, kEpsBlock, sc, sci);
                    s_colscale[tid]              = sc;
                    p.s_col[tm * p.N + tn * kBlk + tid] = sci;
                }
                __syncthreads();
                float2 s2[4];
#pragma unroll
                for (int w = 0; w < 4; ++w) s2[w] = make_float2(s_colscale[tx * 8 + 2 * w], s_colscale[tx * 8 + 2 * w + 1]);
                uint8_t *dst = p.q_col + (out_row0 + ty) * p.N + col;
#pragma unroll
                for (int i = 0; i < 8; ++i) scale_store8_t<FMT, T>(raw[i], s2, dst + i * step);
            }
            return;
        }
    }

    RowFrag<T> frag[8];
    float rmax[8];
    float cmax[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) cmax[j] = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int64_t r = in_row0 + ty + 16 * i;
        if (r < in_end && col < p.N) {
            if constexpr (ACT != 0) frag[i].raw = load_tile8<T, ACT>(xb + r * p.x_ld, col, p.N, p.act_probs[r]); // N % 8 == 0 here
            else frag[i].load(xb + r * p.x_ld, col, p.N, vec_in);
        } else {
            frag[i].zero();
        }
    }
    if constexpr (sizeof(T) == 2) {
        // |x| and max are exact in the storage format, so reduce two elements per instruction there
        using T2 = typename Packed2<T>::type;
        T2 cm2[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) cm2[w] = Packed2<T>::zero();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const T2 *e = reinterpret_cast<const T2 *>(&frag[i].raw);
            T2 a[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                a[w] = __habs2(e[w]);
                if constexpr (MODE & kModeCol) cm2[w] = __hmax2(cm2[w], a[w]);
            }
            const T2 m2 = __hmax2(__hmax2(a[0], a[1]), __hmax2(a[2], a[3]));
            rmax[i]     = fmaxf(to_f32(m2.x), to_f32(m2.y));
        }
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            cmax[2 * w]     = to_f32(cm2[w].x);
            cmax[2 * w + 1] = to_f32(cm2[w].y);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float v[8];
            frag[i].decode(v);
            float m = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float a = fabsf(v[j]);
                m       = fmaxf(m, a);
                if constexpr (MODE & kModeCol) cmax[j] = fmaxf(cmax[j], a);
            }
            rmax[i] = m;
        }
    }

    // ---- row blocks: 16 lanes share a row ---------------------------------------------------
    if constexpr (MODE & kModeRow) {
        uint8_t *qb = p.q_row + b * p.M * p.N;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) rmax[i] = fmaxf(rmax[i], __shfl_xor_sync(0xffffffffu, rmax[i], o));
        }
        // The two IEEE divisions per row are done once, by the lane whose index names the row, and the
        // scale is handed to the other fifteen lanes by shuffle (sixteen redundant divisions per
        // thread were a quarter of the kernel's instructions).
        float mine = rmax[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) mine = ((tx & 7) == i) ? rmax[i] : mine;
        float sc_mine, sci_mine;
        scale_from_amax<FMT>(mine, kEpsBlock, sc_mine, sci_mine);
        const int half_base = (tid & 31) & 16; // first lane of this thread's 16-lane row group
        if (tx < 8) {
            const int64_t r = in_row0 + ty + 16 * tx;
            if (r < in_end) p.s_row[r * p.s_row_stride_m + tn * p.s_row_stride_nb] = sci_mine;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float sc  = __shfl_sync(0xffffffffu, sc_mine, half_base + i);
            const int64_t r = in_row0 + ty + 16 * i;
            if (r < in_end && col < p.N) {
                float qv[8];
                frag[i].decode(qv);
#pragma unroll
                for (int j = 0; j < 8; ++j) qv[j] = quant_val<FMT>(qv[j], sc);
                store8_fp8<FMT>(qb + r * p.N, col, p.N, vec_out, qv);
            }
        }
    }

    // ---- column blocks: reduce the 16 row lanes through shared memory -----------------------
    if constexpr (MODE & kModeCol) {
#pragma unroll
        for (int j = 0; j < 8; ++j) s_colmax[ty][tx * 8 + j] = cmax[j];
        __syncthreads();
        if (tid < kBlk) {
            float m = 0.0f;
#pragma unroll
            for (int k = 0; k < 16; ++k) m = fmaxf(m, s_colmax[k][tid]);
            float sc, sci;
            scale_from_amax<FMT>(m, kEpsBlock, sc, sci);
            s_colscale[tid]  = sc;
            const int64_t c  = tn * kBlk + tid;
            if (c < p.N) p.s_col[tm * p.N + c] = sci;
        }
        __syncthreads();
        float cs[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) cs[j] = s_colscale[tx * 8 + j];
        uint8_t *qb = p.q_col; // column copy exists only for 2-D inputs (B == 1)
        const int64_t out_end = SEGMENT ? (out_row0 + kBlk) : p.M;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int64_t r = out_row0 + ty + 16 * i;
            if (r < out_end && col < p.N) {
                float qv[8];
                frag[i].decode(qv);
#pragma unroll
                for (int j = 0; j < 8; ++j) qv[j] = quant_val<FMT>(qv[j], cs[j]);
                store8_fp8<FMT>(qb + r * p.N, col, p.N, vec_out, qv);
            }
        }
    }

    // ---- whole tile ---------------------------------------------------------------------------
    if constexpr (MODE & kMode2D) {
        float m = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) m = fmaxf(m, rmax[i]);
        m = warp_max(m);
        if ((tid & 31) == 0) s_red[tid >> 5] = m;
        __syncthreads();
        m = s_red[0];
#pragma unroll
        for (int k = 1; k < 8; ++k) m = fmaxf(m, s_red[k]);
        float sc, sci;
        scale_from_amax<FMT>(m, kEpsBlock, sc, sci);
        uint8_t *qb = p.q_row + b * p.M * p.N;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int64_t r = in_row0 + ty + 16 * i;
            if (r < in_end && col < p.N) {
                float qv[8];
                frag[i].decode(qv);
#pragma unroll
                for (int j = 0; j < 8; ++j) qv[j] = quant_val<FMT>(qv[j], sc);
                store8_fp8<FMT>(qb + r * p.N, col, p.N, vec_out, qv);
            }
        }
        if (tid == 0) p.s_2d[(b * tiles_m + tm) * tiles_n + tn] = sci;
    }
}

template <int MODE, bool SEGMENT>
int launch_block_quant(BlockQuantArgs a, int x_dtype, int q_dtype, cudaStream_t st) {
    if (a.x_ld == 0) a.x_ld = a.N;
    const int64_t rows = SEGMENT ? (a.M + a.G * kBlk) : a.M;
    const int64_t tiles_m = cdiv<int64_t>(rows, kBlk) * (SEGMENT ? 1 : a.B);
    const int64_t tiles_n = cdiv<int64_t>(a.N, kBlk);
    if (tiles_m == 0 || tiles_n == 0) return 0;
    PTB_REQUIRE(tiles_n * tiles_m <= 2147483647LL, PTB_ERR_TOO_LARGE, "tile grid too large");
    // every path of the tile kernel writes FP8 with 8-byte stores
    PTB_REQUIRE((reinterpret_cast<uintptr_t>(a.q_row) & 7u) == 0 && (reinterpret_cast<uintptr_t>(a.q_col) & 7u) == 0,
                PTB_ERR_ALIGN, "blockwise quantise: FP8 output pointers must be 8-byte aligned");
    const unsigned grid = (unsigned) (tiles_m * tiles_n);
    PTB_SWITCH_HP(x_dtype, T, PTB_SWITCH_FP8(q_dtype, FMT,
        (quant_block_kernel<T, FMT, MODE, SEGMENT><<<grid, 256, 0, st>>>(a))));
    PTB_LAUNCH_CHECK("quant_block_kernel");
    return 0;
}

// ---- tensorwise -------------------------------------------------------------------------------
template <typename T> __global__ void __launch_bounds__(512) amax_kernel(const T *__restrict__ x, int64_t n,
                                                                          unsigned *amax_bits) {
    __shared__ float s_red[16];
    constexpr int V = 16 / sizeof(T); // elements per 16-byte load
    float m = 0.0f;
    const int64_t nvec = ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) ? n / V : 0;
    const int64_t gtid = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t gsz  = (int64_t) gridDim.x * blockDim.x;
    for (int64_t i = gtid; i < nvec; i += gsz) {
        uint4 raw = reinterpret_cast<const uint4 *>(x)[i];
        const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
        for (int j = 0; j < V; ++j) m = fmaxf(m, fabsf(to_f32(e[j])));
    }
    for (int64_t i = nvec * V + gtid; i < n; i += gsz) m = fmaxf(m, fabsf(to_f32(x[i])));
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        m = (threadIdx.x < (blockDim.x >> 5)) ? s_red[threadIdx.x] : 0.0f;
        m = warp_max(m);
        // non-negative floats order like their bit patterns
        if (threadIdx.x == 0) atomicMax(amax_bits, __float_as_uint(m));
    }
}

// SCALE_GIVEN: `src` holds the scale itself; otherwise it holds the amax bits.
template <typename T, int FMT, bool SCALE_GIVEN>
__global__ void __launch_bounds__(512) quant_tensorwise_kernel(const T *__restrict__ x, int64_t n,
                                                                const float *__restrict__ src,
                                                                uint8_t *__restrict__ q, float *scale_inv) {
    float sc, sci;
    if constexpr (SCALE_GIVEN) {
        sc  = *src;
        sci = __fdiv_rn(1.0f, sc);
    } else {
        scale_from_amax<FMT>(*src, kEpsTensorRow, sc, sci);
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale_inv = sci;
    const bool vec = ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) && ((reinterpret_cast<uintptr_t>(q) & 7u) == 0);
    const int64_t n8   = vec ? n / 8 : 0;
    const int64_t gtid = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t gsz  = (int64_t) gridDim.x * blockDim.x;
    for (int64_t i = gtid; i < n8; i += gsz) {
        float v[8];
        load8<T>(x, i * 8, n, true, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = quant_val<FMT>(v[j], sc);
        store8_fp8<FMT>(q, i * 8, n, true, v);
    }
    for (int64_t i = n8 * 8 + gtid; i < n; i += gsz) q[i] = cvt_fp8<FMT>(quant_val<FMT>(to_f32(x[i]), sc));
}

// ---- rowwise, reduction axis contiguous: one CTA per row, two scans of the row ----------------
template <typename T, int FMT>
__global__ void __launch_bounds__(256) quant_rowwise_inner_kernel(const T *__restrict__ x, int64_t inner,
                                                                   uint8_t *__restrict__ q,
                                                                   float *__restrict__ scale_inv) {
    __shared__ float s_red[8];
    const int64_t row = blockIdx.x;
    const T *xr       = x + row * inner;
    uint8_t *qr       = q + row * inner;
    const bool vec    = (inner % 8 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) &&
                     ((reinterpret_cast<uintptr_t>(q) & 7u) == 0);
    float m = 0.0f;
    for (int64_t c = (int64_t) threadIdx.x * 8; c < inner; c += 256 * 8) {
        float v[8];
        load8<T>(xr, c, inner, vec, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(v[j]));
    }
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = s_red[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) m = fmaxf(m, s_red[k]);
    float sc, sci;
    scale_from_amax<FMT>(m, kEpsTensorRow, sc, sci);
    if (threadIdx.x == 0) scale_inv[row] = sci;
    for (int64_t c = (int64_t) threadIdx.x * 8; c < inner; c += 256 * 8) {
        float v[8];
        load8<T>(xr, c, inner, vec, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = quant_val<FMT>(v[j], sc);
        store8_fp8<FMT>(qr, c, inner, vec, v);
    }
}

// ---- rowwise, reduction axis strided: x [B, M, N], reduce over M ------------------------------
// CTA = 32 column fragments (256 columns) x 8 row lanes, over a chunk of kColChunk rows.
constexpr int kColChunk = 128;

template <typename T>
__global__ void __launch_bounds__(256) col_amax_kernel(const T *__restrict__ x, int64_t M, int64_t N,
                                                        unsigned *__restrict__ amax_bits) {
    __shared__ float s_m[8][256 + 1];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t b   = blockIdx.z;
    const int64_t col = (int64_t) blockIdx.x * 256 + tx * 8;
    const int64_t r0  = (int64_t) blockIdx.y * kColChunk;
    const int64_t r1  = min(r0 + kColChunk, M);
    const T *xb       = x + b * M * N;
    const bool vec    = (N % 8 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15u) == 0);
    float cm[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) cm[j] = 0.0f;
    if (col < N) {
        for (int64_t r = r0 + ty; r < r1; r += 8) {
            float v[8];
            load8<T>(xb + r * N, col, N, vec, v);
#pragma unroll
            for (int j = 0; j < 8; ++j) cm[j] = fmaxf(cm[j], fabsf(v[j]));
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) s_m[ty][tx * 8 + j] = cm[j];
    __syncthreads();
    const int64_t c = (int64_t) blockIdx.x * 256 + threadIdx.x;
    if (c < N) {
        float m = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k) m = fmaxf(m, s_m[k][threadIdx.x]);
        atomicMax(amax_bits + b * N + c, __float_as_uint(m));
    }
}

template <typename T, int FMT>
__global__ void __launch_bounds__(256) quant_rowwise_outer_kernel(const T *__restrict__ x, int64_t M, int64_t N,
                                                                   const float *__restrict__ amax,
                                                                   uint8_t *__restrict__ q,
                                                                   float *__restrict__ scale_inv) {
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t b   = blockIdx.z;
    const int64_t col = (int64_t) blockIdx.x * 256 + tx * 8;
    if (col >= N) return;
    const int64_t r0 = (int64_t) blockIdx.y * kColChunk;
    const int64_t r1 = min(r0 + kColChunk, M);
    const T *xb      = x + b * M * N;
    uint8_t *qb      = q + b * M * N;
    const bool vec   = (N % 8 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) &&
                     ((reinterpret_cast<uintptr_t>(q) & 7u) == 0);
    float sc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float sci = 0.0f;
        sc[j]     = 0.0f;
        if (col + j < N) {
            scale_from_amax<FMT>(amax[b * N + col + j], kEpsTensorRow, sc[j], sci);
            if (blockIdx.y == 0 && ty == 0) scale_inv[b * N + col + j] = sci;
        }
    }
    for (int64_t r = r0 + ty; r < r1; r += 8) {
        float v[8];
        load8<T>(xb + r * N, col, N, vec, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = quant_val<FMT>(v[j], sc[j]);
        store8_fp8<FMT>(qb + r * N, col, N, vec, v);
    }
}

// ---- dequantize: out = cast(float(q) * scale_inv[...]) ----------------------------------------
// q viewed as [B, M, N]; scale index = b*sb + (m / bm)*sm + (n / bn)*sn.
struct DequantIdx {
    int64_t M, N;
    int64_t sb, bm, sm, bn, sn;
};

template <typename TO, int FMT>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t *__restrict__ q, int64_t n,
                                                       const float *__restrict__ scale_inv, DequantIdx ix,
                                                       TO *__restrict__ out) {
    const int64_t gtid = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t gsz  = (int64_t) gridDim.x * blockDim.x;
    for (int64_t i = gtid; i < n; i += gsz) {
        const int64_t col = i % ix.N;
        const int64_t rw  = i / ix.N;
        const int64_t m = rw % ix.M, b = rw / ix.M;
        const int64_t si = b * ix.sb + (m / ix.bm) * ix.sm + (col / ix.bn) * ix.sn;
        out[i]           = from_f32<TO>(fp8_to_f32<FMT>(q[i]) * scale_inv[si]);
    }
}

// Vector form: one thread dequantises 16 consecutive elements of a row (one 16-byte load of FP8, 32 or 64
// bytes of output), the row / column split is done once per vector instead of once per element, and the
// scale is either one value for the whole vector (column blocks of 16 or more) or 16 consecutive
// values (one scale per column).  Used whenever N is a multiple of 16 and the buffers are aligned.
template <typename TO, int FMT, bool PER_COLUMN>
__global__ void __launch_bounds__(256) dequant_vec_kernel(const uint8_t *__restrict__ q, int64_t nvec,
                                                           const float *__restrict__ scale_inv, DequantIdx ix,
                                                           TO *__restrict__ out) {
    const int64_t vec_per_row = ix.N / 16;
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t) gridDim.x * blockDim.x) {
        const int64_t rw = i / vec_per_row, col = (i - rw * vec_per_row) * 16;
        const int64_t m = rw % ix.M, b = rw / ix.M;
        const int64_t si = b * ix.sb + (m / ix.bm) * ix.sm + (col / ix.bn) * ix.sn;
        const uint4 raw  = *reinterpret_cast<const uint4 *>(q + i * 16);
        const uint8_t *e = reinterpret_cast<const uint8_t *>(&raw);
        float sc[16];
        if constexpr (PER_COLUMN) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float4 s4 = *reinterpret_cast<const float4 *>(scale_inv + si + 4 * k);
                sc[4 * k] = s4.x; sc[4 * k + 1] = s4.y; sc[4 * k + 2] = s4.z; sc[4 * k + 3] = s4.w;
            }
        } else {
            const float s1 = scale_inv[si];
#pragma unroll
            for (int k = 0; k < 16; ++k) sc[k] = s1;
        }
        TO o[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) o[k] = from_f32<TO>(fp8_to_f32<FMT>(e[k]) * sc[k]);
        uint4 *dst = reinterpret_cast<uint4 *>(out + i * 16);
#pragma unroll
        for (int k = 0; k < (int) (sizeof(TO) * 16 / 16); ++k) dst[k] = reinterpret_cast<const uint4 *>(o)[k];
    }
}

int launch_dequant(const void *q, int q_dtype, int64_t n, const float *s, const DequantIdx &ix, void *out,
                   int out_dtype, cudaStream_t st) {
    if (n == 0) return 0;
    PTB_REQUIRE(q && s && out, PTB_ERR_ARG, "dequant: null pointer");
    PTB_REQUIRE(is_hp(out_dtype) && is_fp8(q_dtype), PTB_ERR_ARG, "dequant: bad dtype");
    const bool per_column = ix.bn == 1 && ix.sn == 1;
    const bool one_scale  = ix.sn == 0 || (ix.bn >= 16 && ix.bn % 16 == 0);
    if (ix.N % 16 == 0 && (per_column || one_scale) && aligned16(q) && aligned16(out) &&
        (!per_column || (aligned16(s) && ix.sb % 4 == 0 && ix.sm % 4 == 0))) {
        const int64_t nvec = n / 16;
        const int blocks   = (int) imin(cdiv<int64_t>(nvec, 256), 148 * 32);
        if (per_column) {
            PTB_SWITCH_HP(out_dtype, TO, PTB_SWITCH_FP8(q_dtype, FMT,
                (dequant_vec_kernel<TO, FMT, true><<<blocks, 256, 0, st>>>((const uint8_t *) q, nvec, s, ix, (TO *) out))));
        } else {
            PTB_SWITCH_HP(out_dtype, TO, PTB_SWITCH_FP8(q_dtype, FMT,
                (dequant_vec_kernel<TO, FMT, false><<<blocks, 256, 0, st>>>((const uint8_t *) q, nvec, s, ix, (TO *) out))));
        }
        PTB_LAUNCH_CHECK("dequant_vec_kernel");
        return 0;
    }
    const int blocks = (int) imin(cdiv<int64_t>(n, 256), 148 * 16);
    PTB_SWITCH_HP(out_dtype, TO, PTB_SWITCH_FP8(q_dtype, FMT,
        (dequant_kernel<TO, FMT><<<blocks, 256, 0, st>>>((const uint8_t *) q, n, s, ix, (TO *) out))));
    PTB_LAUNCH_CHECK("dequant_kernel");
    return 0;
}

// ---- exclusive prefix sum of group lengths ------------------------------------------------------
__global__ void __launch_bounds__(256) group_offs_kernel(const int64_t *__restrict__ lens, int64_t G,
                                                          int64_t *__restrict__ offs) {
    __shared__ int64_t s_scan[256];
    const int tid     = threadIdx.x;
    const int64_t per = cdiv<int64_t>(G, 256);
    const int64_t g0 = (int64_t) tid * per, g1 = min(g0 + per, G);
    int64_t local = 0;
    for (int64_t g = g0; g < g1; ++g) local += lens[g];
    s_scan[tid] = local;
    __syncthreads();
    for (int off = 1; off < 256; off <<= 1) {
        int64_t add = (tid >= off) ? s_scan[tid - off] : 0;
        __syncthreads();
        s_scan[tid] += add;
        __syncthreads();
    }
    int64_t run = s_scan[tid] - local;
    for (int64_t g = g0; g < g1; ++g) {
        offs[g] = run;
        run += lens[g];
    }
    if (tid == 255) offs[G] = s_scan[255];
}

// ---- byte transpose [B, M, N] -> [B, N, M] ------------------------------------------------------
__global__ void __launch_bounds__(256) transpose_u8_kernel(const uint8_t *__restrict__ in, int64_t M, int64_t N,
                                                            uint8_t *__restrict__ out) {
    __shared__ uint8_t tile[64][64 + 4];
    const int64_t b  = blockIdx.z;
    const int64_t m0 = (int64_t) blockIdx.y * 64, n0 = (int64_t) blockIdx.x * 64;
    const uint8_t *ib = in + b * M * N;
    uint8_t *ob       = out + b * M * N;
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6; // 64 x 4
    for (int r = ty; r < 64; r += 4) {
        int64_t m = m0 + r, n = n0 + tx;
        tile[r][tx] = (m < M && n < N) ? ib[m * N + n] : (uint8_t) 0;
    }
    __syncthreads();
    for (int r = ty; r < 64; r += 4) {
        int64_t n = n0 + r, m = m0 + tx;
        if (n < N && m < M) ob[n * M + m] = tile[tx][r];
    }
}

} // namespace
} // namespace ptb

using namespace ptb;

// =================================================================================================
// C entry points
// =================================================================================================
extern "C" {
#pragma GCC visibility push(default)

int ptb_version(void) { return PTB_VERSION; }
const char *ptb_last_error(void) { return err_buf(); }

int ptb_quant_fp8_tensorwise(const void *x, int x_dtype, int64_t n, void *q, int q_dtype, float *scale_inv,
                             void *workspace, ptb_stream_t stream) {
    PTB_REQUIRE(n >= 0, PTB_ERR_ARG, "quant_tensorwise: n < 0");
    PTB_REQUIRE(scale_inv && workspace, PTB_ERR_ARG, "quant_tensorwise: null scale_inv/workspace");
    PTB_REQUIRE(n == 0 || (x && q), PTB_ERR_ARG, "quant_tensorwise: null x/q");
    PTB_REQUIRE(is_hp(x_dtype) && is_fp8(q_dtype), PTB_ERR_ARG, "quant_tensorwise: bad dtype");
    cudaStream_t st = (cudaStream_t) stream;
    PTB_CUDA(cudaMemsetAsync(workspace, 0, sizeof(unsigned), st));
    const int blocks = (int) imax(1, imin(cdiv<int64_t>(n, 512 * 8), 148 * 4));
    if (n > 0) {
        PTB_SWITCH_HP(x_dtype, T, (amax_kernel<T><<<blocks, 512, 0, st>>>((const T *) x, n, (unsigned *) workspace)));
        PTB_LAUNCH_CHECK("amax_kernel");
    }
    PTB_SWITCH_HP(x_dtype, T, PTB_SWITCH_FP8(q_dtype, FMT,
        (quant_tensorwise_kernel<T, FMT, false><<<blocks, 512, 0, st>>>((const T *) x, n, (const float *) workspace,
                                                                         (uint8_t *) q, scale_inv))));
    PTB_LAUNCH_CHECK("quant_tensorwise_kernel");
    return 0;
}

int ptb_quant_fp8_tensorwise_with_scale(const void *x, int x_dtype, int64_t n, const float *scale, void *q,
                                        int q_dtype, float *scale_inv, ptb_stream_t stream) {
    PTB_REQUIRE(n >= 0 && scale && scale_inv, PTB_ERR_ARG, "quant_tensorwise_with_scale: bad argument");
    PTB_REQUIRE(n == 0 || (x && q), PTB_ERR_ARG, "quant_tensorwise_with_scale: null x/q");
    PTB_REQUIRE(is_hp(x_dtype) && is_fp8(q_dtype), PTB_ERR_ARG, "quant_tensorwise_with_scale: bad dtype");
    cudaStream_t st  = (cudaStream_t) stream;
    const int blocks = (int) imax(1, imin(cdiv<int64_t>(n, 512 * 8), 148 * 4));
    PTB_SWITCH_HP(x_dtype, T, PTB_SWITCH_FP8(q_dtype, FMT,
        (quant_tensorwise_kernel<T, FMT, true><<<blocks, 512, 0, st>>>((const T *) x, n, scale, (uint8_t *) q,
                                                                        scale_inv))));
    PTB_LAUNCH_CHECK("quant_tensorwise_kernel");
    return 0;
}

int ptb_quant_fp8_rowwise(const void *x, int x_dtype, int64_t B, int64_t M, int64_t N, void *q, int q_dtype,
                          float *scale_inv, void *workspace, ptb_stream_t stream) {
    PTB_REQUIRE(B >= 0 && M >= 0 && N >= 0, PTB_ERR_ARG, "quant_rowwise: negative size");
    PTB_REQUIRE(is_hp(x_dtype) && is_fp8(q_dtype), PTB_ERR_ARG, "quant_rowwise: bad dtype");
    if (B * N == 0) return 0;
    PTB_REQUIRE(scale_inv, PTB_ERR_ARG, "quant_rowwise: null scale_inv");
    PTB_REQUIRE(M == 0 || (x && q), PTB_ERR_ARG, "quant_rowwise: null x/q");
    cudaStream_t st = (cudaStream_t) stream;
    if (N == 1) {
        PTB_REQUIRE(B <= 2147483647LL, PTB_ERR_TOO_LARGE, "quant_rowwise: too many rows");
        PTB_SWITCH_HP(x_dtype, T, PTB_SWITCH_FP8(q_dtype, FMT,
            (quant_rowwise_inner_kernel<T, FMT><<<(unsigned) B, 256, 0, st>>>((const T *) x, M, (uint8_t *) q,
                                                                               scale_inv))));
        PTB_LAUNCH_CHECK("quant_rowwise_inner_kernel");
        return 0;
    }
    PTB_REQUIRE(workspace, PTB_ERR_ARG, "quant_rowwise: null workspace");
    PTB_REQUIRE(B <= 65535 && cdiv<int64_t>(M, kColChunk) <= 65535, PTB_ERR_TOO_LARGE, "quant_rowwise: grid too large");
    PTB_CUDA(cudaMemsetAsync(workspace, 0, sizeof(float) * B * N, st));
    dim3 grid((unsigned) cdiv<int64_t>(N, 256), (unsigned) imax(1, cdiv<int64_t>(M, kColChunk)), (unsigned) B);
    PTB_SWITCH_HP(x_dtype, T, (col_amax_kernel<T><<<grid, 256, 0, st>>>((const T *) x, M, N, (unsigned *) workspace)));
    PTB_LAUNCH_CHECK("col_amax_kernel");
    PTB_SWITCH_HP(x_dtype, T, PTB_SWITCH_FP8(q_dtype, FMT,
        (quant_rowwise_outer_kernel<T, FMT><<<grid, 256, 0, st>>>((const T *) x, M, N, (const float *) workspace,
                                                                   (uint8_t *) q, scale_inv))));
    PTB_LAUNCH_CHECK("quant_rowwise_outer_kernel");
    return 0;
}

// ---- rowwise quantize for callers that may not allocate ------------------------------------------
// The column-amax scratch of the strided rowwise path lives in this fixed array instead of a
// caller-provided workspace.  Every GPU that loads the library carries these 256 KiB until exit.
#define PTB_NOALLOC_MAX_COLUMNS 65536
static __device__ __align__(256) float g_noalloc_rowwise_scratch[PTB_NOALLOC_MAX_COLUMNS];

// Device address of the array above on the current device.  The array's name is only a host-side
// handle here, so the address is asked for once per device and remembered.  The cache entries are
// atomics: two host threads that make a device's first call together both look the address up and
// store the same value.  A cudaDeviceReset invalidates the cache; a process that resets a device
// must not call this entry point on it afterwards.
static int noalloc_scratch_address(float **out) {
    static std::atomic<float *> address_on_device[64];
    int dev = -1;
    PTB_CUDA(cudaGetDevice(&dev));
    PTB_REQUIRE(dev >= 0 && dev < 64, PTB_ERR_UNSUPPORTED, "quant_rowwise_noalloc: device index %d not supported", dev);
    float *p = address_on_device[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        PTB_CUDA(cudaGetSymbolAddress((void **) &p, g_noalloc_rowwise_scratch));
        PTB_REQUIRE(p != nullptr, PTB_ERR_DRIVER, "quant_rowwise_noalloc: scratch array has no device address");
        address_on_device[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return 0;
}

int ptb_quant_fp8_rowwise_noalloc(const void *x, int x_dtype, int64_t B, int64_t M, int64_t N, void *q, int q_dtype,
                                  float *scale_inv, ptb_stream_t stream) {
    PTB_REQUIRE(B >= 0 && M >= 0 && N >= 0, PTB_ERR_ARG, "quant_rowwise_noalloc: negative size");
    // N == 1 (the reduction axis is the innermost one) reduces inside one CTA and uses no scratch
    if (N == 1) return ptb_quant_fp8_rowwise(x, x_dtype, B, M, N, q, q_dtype, scale_inv, nullptr, stream);
    // bound each factor before multiplying: the product of two huge sizes could wrap
    PTB_REQUIRE(B <= (int64_t) PTB_NOALLOC_MAX_COLUMNS && N <= (int64_t) PTB_NOALLOC_MAX_COLUMNS &&
                    B * N <= (int64_t) PTB_NOALLOC_MAX_COLUMNS,
                PTB_ERR_TOO_LARGE,
                "quant_rowwise_noalloc: B = %lld times N = %lld scale columns exceed the built-in scratch of %d; "
                "use ptb_quant_fp8_rowwise with a caller-provided workspace",
                (long long) B, (long long) N, PTB_NOALLOC_MAX_COLUMNS);
    float *scratch = nullptr;
    int rc = noalloc_scratch_address(&scratch);
    if (rc) return rc;
    // same kernels as the workspace variant; it clears the B*N scratch words it uses before reducing into them
    return ptb_quant_fp8_rowwise(x, x_dtype, B, M, N, q, q_dtype, scale_inv, scratch, stream);
}

int ptb_quant_fp8_block1d(const void *x, int x_dtype, int64_t M, int64_t N, int axis, void *q, int q_dtype,
                          float *scale_inv, ptb_stream_t stream) {
    PTB_REQUIRE(M >= 0 && N >= 0 && (axis == 0 || axis == 1), PTB_ERR_ARG, "quant_block1d: bad size/axis");
    if (M * N == 0) return 0;
    PTB_REQUIRE(x && q && scale_inv, PTB_ERR_ARG, "quant_block1d: null pointer");
    BlockQuantArgs a{};
    a.x = x; a.B = 1; a.M = M; a.N = N;
    if (axis == 1) {
        a.q_row = (uint8_t *) q; a.s_row = scale_inv;
        a.s_row_stride_m = cdiv<int64_t>(N, kBlk); a.s_row_stride_nb = 1;
        return launch_block_quant<kModeRow, false>(a, x_dtype, q_dtype, (cudaStream_t) stream);
    }
    a.q_col = (uint8_t *) q; a.s_col = scale_inv;
    return launch_block_quant<kModeCol, false>(a, x_dtype, q_dtype, (cudaStream_t) stream);
}

int ptb_quant_fp8_block1d_dual(const void *x, int x_dtype, int64_t M, int64_t N, void *q_row, float *s_row,
                               void *q_col, float *s_col, int q_dtype, ptb_stream_t stream) {
    PTB_REQUIRE(M >= 0 && N >= 0, PTB_ERR_ARG, "quant_block1d_dual: negative size");
    if (M * N == 0) return 0;
    PTB_REQUIRE(x && q_row && s_row && q_col && s_col, PTB_ERR_ARG, "quant_block1d_dual: null pointer");
    BlockQuantArgs a{};
    a.x = x; a.B = 1; a.M = M; a.N = N;
    a.q_row = (uint8_t *) q_row; a.s_row = s_row;
    a.s_row_stride_m = cdiv<int64_t>(N, kBlk); a.s_row_stride_nb = 1;
    a.q_col = (uint8_t *) q_col; a.s_col = s_col;
    return launch_block_quant<kModeRow | kModeCol, false>(a, x_dtype, q_dtype, (cudaStream_t) stream);
}

int ptb_quant_fp8_block2d(const void *w, int w_dtype, int64_t B, int64_t M, int64_t N, void *q, int q_dtype,
                          float *scale_inv, ptb_stream_t stream) {
    PTB_REQUIRE(B >= 0 && M >= 0 && N >= 0, PTB_ERR_ARG, "quant_block2d: negative size");
    if (B * M * N == 0) return 0;
    PTB_REQUIRE(w && q && scale_inv, PTB_ERR_ARG, "quant_block2d: null pointer");
    BlockQuantArgs a{};
    a.x = w; a.B = B; a.M = M; a.N = N;
    a.q_row = (uint8_t *) q; a.s_2d = scale_inv;
    return launch_block_quant<kMode2D, false>(a, w_dtype, q_dtype, (cudaStream_t) stream);
}

int ptb_quant_fp8_segment_row_col(const void *x, int x_dtype, int64_t M, int64_t N, int64_t G,
                                  const int64_t *group_lens, const int64_t *group_offs, void *q_row,
                                  void *q_col_padded, float *s_row, float *s_col_padded, int64_t *var_k_lens,
                                  int64_t *var_k_offs, void *block_table, int q_dtype, ptb_stream_t stream) {
    (void) group_lens; // lengths are implied by the offsets
    PTB_REQUIRE(M >= 0 && N >= 0 && G >= 0, PTB_ERR_ARG, "quant_segment_row_col: negative size");
    PTB_REQUIRE(group_offs && var_k_lens && var_k_offs, PTB_ERR_ARG, "quant_segment_row_col: null group arrays");
    PTB_REQUIRE(N > 0, PTB_ERR_ARG, "quant_segment_row_col: N must be positive");
    // a rank of an expert-parallel job may receive no row at all: the tensors with M rows are then empty
    // (null), the padded layout is still written (all groups empty) and nothing else happens
    PTB_REQUIRE(M == 0 || (x && q_row && s_row), PTB_ERR_ARG, "quant_segment_row_col: null pointer");
    PTB_REQUIRE(M + G == 0 || (q_col_padded && s_col_padded), PTB_ERR_ARG, "quant_segment_row_col: null pointer");
    BlockQuantArgs a{};
    a.x = x; a.B = 1; a.M = M; a.N = N; a.G = G;
    a.q_row = (uint8_t *) q_row; a.s_row = s_row;
    a.s_row_stride_m = 1; a.s_row_stride_nb = M; // row scales stored [ceil(N/128), M]
    a.q_col = (uint8_t *) q_col_padded; a.s_col = s_col_padded;
    a.group_offs = group_offs; a.var_k_offs = var_k_offs;
    PTB_REQUIRE(block_table == nullptr || M < 2147483647LL, PTB_ERR_TOO_LARGE,
                "quant_segment_row_col: the block table holds 32-bit row numbers");
    a.block_table = (const int2 *) block_table;
    segment_offsets_kernel<<<1, 256, 0, (cudaStream_t) stream>>>(group_offs, G, var_k_lens, var_k_offs,
                                                                  (int2 *) block_table);
    PTB_LAUNCH_CHECK("segment_offsets_kernel");
    if (M == 0) return 0;
    // the activation / grad-out shapes of the MoE path: 16-bit, whole column tiles, aligned rows, a block table
    if (PTB_SEG_STREAM && block_table != nullptr && (x_dtype == PTB_BF16 || x_dtype == PTB_F16) && N % kBlk == 0 && aligned16(x) &&
        (reinterpret_cast<uintptr_t>(q_row) & 7u) == 0 && (reinterpret_cast<uintptr_t>(q_col_padded) & 7u) == 0) {
        const int64_t tiles_m = cdiv<int64_t>(M + G * kBlk, kBlk);
        const int64_t strips  = cdiv<int64_t>(N / kBlk, kSegStrip);
        PTB_REQUIRE(tiles_m * strips <= 2147483647LL, PTB_ERR_TOO_LARGE, "tile grid too large");
        const unsigned grid = (unsigned) (tiles_m * strips);
        cudaStream_t st     = (cudaStream_t) stream;
        if (x_dtype == PTB_BF16) {
            PTB_SWITCH_FP8(q_dtype, FMT, (seg_quant_stream_kernel<__nv_bfloat16, FMT><<<grid, 256, 0, st>>>(a)));
        } else {
            PTB_SWITCH_FP8(q_dtype, FMT, (seg_quant_stream_kernel<__half, FMT><<<grid, 256, 0, st>>>(a)));
        }
        PTB_LAUNCH_CHECK("seg_quant_stream_kernel");
        return 0;
    }
    return launch_block_quant<kModeRow | kModeCol, true>(a, x_dtype, q_dtype, (cudaStream_t) stream);
}

int ptb_swiglu_quant_fp8_segment_row_col(const void *x, int x_dtype, const float *probs, int64_t M, int64_t N, int64_t G,
                                         const int64_t *group_offs, void *q_row, void *q_col_padded, float *s_row,
                                         float *s_col_padded, int64_t *var_k_lens, int64_t *var_k_offs,
                                         void *block_table, int q_dtype, ptb_stream_t stream) {
    PTB_REQUIRE(M >= 0 && N > 0 && G >= 0, PTB_ERR_ARG, "swiglu_quant_segment_row_col: bad size");
    PTB_REQUIRE(N % 8 == 0, PTB_ERR_ALIGN, "swiglu_quant_segment_row_col: the hidden size must be a multiple of 8");
    PTB_REQUIRE(x_dtype == PTB_BF16 || x_dtype == PTB_F16, PTB_ERR_ARG, "swiglu_quant_segment_row_col: x must be bf16 or fp16");
    PTB_REQUIRE(group_offs && var_k_lens && var_k_offs, PTB_ERR_ARG, "swiglu_quant_segment_row_col: null group arrays");
    PTB_REQUIRE(M == 0 || (x && probs && q_row && s_row), PTB_ERR_ARG, "swiglu_quant_segment_row_col: null pointer");
    PTB_REQUIRE(M + G == 0 || (q_col_padded && s_col_padded), PTB_ERR_ARG, "swiglu_quant_segment_row_col: null pointer");
    PTB_REQUIRE(aligned16(x), PTB_ERR_ALIGN, "swiglu_quant_segment_row_col: x must be 16-byte aligned");
    PTB_REQUIRE(block_table == nullptr || M < 2147483647LL, PTB_ERR_TOO_LARGE,
                "swiglu_quant_segment_row_col: the block table holds 32-bit row numbers");
    BlockQuantArgs a{};
    a.x = x; a.B = 1; a.M = M; a.N = N; a.G = G; a.x_ld = 2 * N; a.act_probs = probs;
    a.q_row = (uint8_t *) q_row; a.s_row = s_row;
    a.s_row_stride_m = 1; a.s_row_stride_nb = M;
    a.q_col = (uint8_t *) q_col_padded; a.s_col = s_col_padded;
    a.group_offs = group_offs; a.var_k_offs = var_k_offs; a.block_table = (const int2 *) block_table;
    cudaStream_t st = (cudaStream_t) stream;
    segment_offsets_kernel<<<1, 256, 0, st>>>(group_offs, G, var_k_lens, var_k_offs, (int2 *) block_table);
    PTB_LAUNCH_CHECK("segment_offsets_kernel");
    if (M == 0) return 0;
    const int64_t tiles_m = cdiv<int64_t>(M + G * kBlk, kBlk), tiles_n = cdiv<int64_t>(N, kBlk);
    PTB_REQUIRE(tiles_n * tiles_m <= 2147483647LL, PTB_ERR_TOO_LARGE, "tile grid too large");
    PTB_REQUIRE((reinterpret_cast<uintptr_t>(a.q_row) & 7u) == 0 && (reinterpret_cast<uintptr_t>(a.q_col) & 7u) == 0,
                PTB_ERR_ALIGN, "blockwise quantise: FP8 output pointers must be 8-byte aligned");
    const unsigned grid = (unsigned) (tiles_m * tiles_n);
    if (x_dtype == PTB_BF16) {
        PTB_SWITCH_FP8(q_dtype, FMT, (quant_block_kernel<__nv_bfloat16, FMT, kModeRow | kModeCol, true, 1><<<grid, 256, 0, st>>>(a)));
    } else {
        PTB_SWITCH_FP8(q_dtype, FMT, (quant_block_kernel<__half, FMT, kModeRow | kModeCol, true, 1><<<grid, 256, 0, st>>>(a)));
    }
    PTB_LAUNCH_CHECK("quant_block_kernel");
    return 0;
}

int ptb_dequant_fp8_tensorwise(const void *q, int q_dtype, int64_t n, const float *scale_inv, void *out,
                               int out_dtype, ptb_stream_t stream) {
    PTB_REQUIRE(n >= 0, PTB_ERR_ARG, "dequant_tensorwise: n < 0");
    DequantIdx ix{1, n > 0 ? n : 1, 0, 1, 0, INT64_MAX, 0};
    return launch_dequant(q, q_dtype, n, scale_inv, ix, out, out_dtype, (cudaStream_t) stream);
}

int ptb_dequant_fp8_rowwise(const void *q, int q_dtype, int64_t B, int64_t M, int64_t N, const float *scale_inv,
                            void *out, int out_dtype, ptb_stream_t stream) {
    PTB_REQUIRE(B >= 0 && M >= 0 && N >= 0, PTB_ERR_ARG, "dequant_rowwise: negative size");
    if (B * M * N == 0) return 0;
    if (N == 1) {
        // the scaled axis is the innermost one: B rows of M elements, one scale per row
        DequantIdx rows{B, M, 0, 1, 1, INT64_MAX, 0}; // scale[m]
        return launch_dequant(q, q_dtype, B * M, scale_inv, rows, out, out_dtype, (cudaStream_t) stream);
    }
    DequantIdx ix{M, N, N, INT64_MAX, 0, 1, 1}; // scale[b, 0, n]
    return launch_dequant(q, q_dtype, B * M * N, scale_inv, ix, out, out_dtype, (cudaStream_t) stream);
}

int ptb_dequant_fp8_block1d(const void *q, int q_dtype, int64_t M, int64_t N, int axis, const float *scale_inv,
                            void *out, int out_dtype, ptb_stream_t stream) {
    PTB_REQUIRE(M >= 0 && N >= 0 && (axis == 0 || axis == 1), PTB_ERR_ARG, "dequant_block1d: bad size/axis");
    if (M * N == 0) return 0;
    DequantIdx ix = (axis == 1) ? DequantIdx{M, N, 0, 1, cdiv<int64_t>(N, kBlk), kBlk, 1}  // scale[m, n/128]
                                : DequantIdx{M, N, 0, kBlk, N, 1, 1};                        // scale[m/128, n]
    return launch_dequant(q, q_dtype, M * N, scale_inv, ix, out, out_dtype, (cudaStream_t) stream);
}

int ptb_dequant_fp8_block2d(const void *q, int q_dtype, int64_t B, int64_t M, int64_t N, const float *scale_inv,
                            void *out, int out_dtype, ptb_stream_t stream) {
    PTB_REQUIRE(B >= 0 && M >= 0 && N >= 0, PTB_ERR_ARG, "dequant_block2d: negative size");
    if (B * M * N == 0) return 0;
    const int64_t mb = cdiv<int64_t>(M, kBlk), nb = cdiv<int64_t>(N, kBlk);
    DequantIdx ix{M, N, mb * nb, kBlk, nb, kBlk, 1}; // scale[b, m/128, n/128]
    return launch_dequant(q, q_dtype, B * M * N, scale_inv, ix, out, out_dtype, (cudaStream_t) stream);
}

int ptb_group_offs(const int64_t *group_lens, int64_t G, int64_t *group_offs, ptb_stream_t stream) {
    PTB_REQUIRE(G >= 0 && group_offs && (G == 0 || group_lens), PTB_ERR_ARG, "group_offs: bad argument");
    group_offs_kernel<<<1, 256, 0, (cudaStream_t) stream>>>(group_lens, G, group_offs);
    PTB_LAUNCH_CHECK("group_offs_kernel");
    return 0;
}

int ptb_transpose_2d_u8(const void *in, int64_t B, int64_t M, int64_t N, void *out, ptb_stream_t stream) {
    PTB_REQUIRE(B >= 0 && M >= 0 && N >= 0, PTB_ERR_ARG, "transpose_2d_u8: negative size");
    if (B * M * N == 0) return 0;
    PTB_REQUIRE(in && out, PTB_ERR_ARG, "transpose_2d_u8: null pointer");
    PTB_REQUIRE(B <= 65535 && cdiv<int64_t>(M, 64) <= 65535, PTB_ERR_TOO_LARGE, "transpose_2d_u8: grid too large");
    dim3 grid((unsigned) cdiv<int64_t>(N, 64), (unsigned) cdiv<int64_t>(M, 64), (unsigned) B);
    transpose_u8_kernel<<<grid, 256, 0, (cudaStream_t) stream>>>((const uint8_t *) in, M, N, (uint8_t *) out);
    PTB_LAUNCH_CHECK("transpose_u8_kernel");
    return 0;
}

#pragma GCC visibility pop
} // extern "C"
