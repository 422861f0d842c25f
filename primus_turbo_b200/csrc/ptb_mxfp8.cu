// MXFP8 quantise / dequantise for sm_100a: 1x32 (or 32x32) blocks with power-of-two E8M0 scales.
//
// Semantics follow the reference's csrc/kernels/quantization/quantization_mxfp8.cu (scale from the block
// maximum: lines 71-110; 32x32 tiles, zero fill outside the matrix, clamp to +-(fmax * scale) then divide
// by the scale: lines 128-515) and dequantization_mxfp8.cu:47-100.  Layouts follow
// csrc/pytorch/quantization/quantization.cpp:736-966: the row-direction output is [M, N_pad], the
// column-direction output is stored TRANSPOSED as [N, M_pad], padded extents are multiples of 128 and
// hold zero bytes with scale byte 0, scales are one byte per 32 elements along the padded extent.
//
// One pass over the input produces both directions.  A warp owns a 32-row x 64-column tile and never
// talks to another warp: row maxima reduce over the four lanes of a 32-column block, column maxima over
// the four lanes that share a column, and the transposed output is assembled with a 4x4 byte transpose
// across those four lanes, so every lane ends up holding 32 contiguous output bytes of two columns.
#include "ptb_common.cuh"

// resident CTAs per SM the quantise kernel is compiled for (measured on 16384 x 8192 bf16, both directions:
// 2 -> 3.3 TB/s without spills, 3 -> 2.8 TB/s and 4 -> 2.6 TB/s with spills)
#ifndef PTB_MXQ_MINB
#define PTB_MXQ_MINB 2
#endif

namespace ptb {
namespace {

constexpr int kMxBlock = 32;
constexpr int kMxPad   = 128;

template <int FMT> struct MxFmt;
template <> struct MxFmt<PTB_E4M3> { static constexpr int mbits = 3, target_pow2 = 8; };
template <> struct MxFmt<PTB_E5M2> { static constexpr int mbits = 2, target_pow2 = 15; };

// Block maximum -> biased E8M0 byte.  The maximum's mantissa is rounded to the FP8 format's width (the
// carry may bump the exponent), the exponent of the format's largest power of two is subtracted, the
// result is clamped to [-127, 128] and biased by 127.
template <int FMT> __device__ __forceinline__ int mx_biased_exponent(float amax) {
    const uint32_t bits = __float_as_uint(amax);
    const int add       = 1 << (23 - MxFmt<FMT>::mbits - 1);
    int e               = (int) (((bits + (uint32_t) add) >> 23) & 0x1ffu) - 127 - MxFmt<FMT>::target_pow2;
    e                   = max(e, -127);
    e                   = min(e, 128);
    return e + 127;
}
template <int FMT, bool ZERO_IS_ONE> __device__ __forceinline__ int mx_byte(float amax) {
    if (ZERO_IS_ONE && amax == 0.0f) return 127;
    return mx_biased_exponent<FMT>(amax);
}
// The reference clamps a value to +-(fmax * scale), scale = (byte << 23) read as fp32, and divides by the
// scale.  Here: multiply by the exact reciprocal 2^(127 - byte) (subnormal for bytes 254 and 255) and let the
// saturating conversion clamp -- the same result for every finite value, because fmax * scale times the
// reciprocal is exactly fmax.  Byte 0 is the one exception: its scale reads as 0.0f, the clamp limit is zero
// and every value becomes +-0, which a multiplier of zero reproduces (sign included).
__device__ __forceinline__ float mx_inverse(int biased) {
    const int e = 127 - biased; // 127 .. -128
    if (biased == 0) return 0.0f;
    return (e >= -126) ? __uint_as_float((uint32_t) (e + 127) << 23) : __uint_as_float(1u << (149 + e));
}

struct MxQuantArgs {
    const void *x;
    uint8_t *q_row, *s_row, *q_col, *s_col;
    int64_t M, N, M_pad, N_pad;
    int row_2d, col_2d;
    // grouped mode: per 128-row block of the padded column layout {first source row, end of the group's
    // source rows, row of the row-direction output that the first source row goes to, group}
    const int4 *table;
};

// Grouped layouts (csrc/pytorch/quantization/quantization.cpp:1100-1130 in the reference): every group's rows
// padded to `row_align` rows in the row-direction output and to 128 rows in the column-direction output.
// One CTA: padded lengths and offsets of both layouts and the block table of MxQuantArgs; blocks past the
// last group get an empty entry (they are written as zeros).
__global__ void __launch_bounds__(256) mx_group_layout_kernel(const int64_t *__restrict__ group_offs, int64_t G, int64_t row_align,
                                                              int64_t *__restrict__ row_lens, int64_t *__restrict__ row_offs,
                                                              int64_t *__restrict__ col_lens, int64_t *__restrict__ col_offs,
                                                              int4 *__restrict__ table, int64_t nblocks) {
    __shared__ int64_t s_row[256], s_col[256];
    const int tid     = threadIdx.x;
    const int64_t per = cdiv<int64_t>(G, 256);
    const int64_t g0 = (int64_t) tid * per, g1 = imin(g0 + per, G);
    int64_t lr = 0, lc = 0;
    for (int64_t g = g0; g < g1; ++g) {
        const int64_t len = group_offs[g + 1] - group_offs[g];
        lr += cdiv<int64_t>(len, row_align) * row_align;
        lc += cdiv<int64_t>(len, kMxPad) * kMxPad;
    }
    s_row[tid] = lr;
    s_col[tid] = lc;
    __syncthreads();
    for (int off = 1; off < 256; off <<= 1) {
        const int64_t ar = (tid >= off) ? s_row[tid - off] : 0, ac = (tid >= off) ? s_col[tid - off] : 0;
        __syncthreads();
        s_row[tid] += ar;
        s_col[tid] += ac;
        __syncthreads();
    }
    int64_t run_r = s_row[tid] - lr, run_c = s_col[tid] - lc;
    for (int64_t g = g0; g < g1; ++g) {
        const int64_t gs = group_offs[g], ge = group_offs[g + 1];
        const int64_t pr = cdiv<int64_t>(ge - gs, row_align) * row_align, pc = cdiv<int64_t>(ge - gs, kMxPad) * kMxPad;
        row_lens[g] = pr; row_offs[g] = run_r;
        col_lens[g] = pc; col_offs[g] = run_c;
        for (int64_t t = 0; t < pc / kMxPad; ++t)
            table[run_c / kMxPad + t] = make_int4((int) (gs + t * kMxPad), (int) ge, (int) (run_r + t * kMxPad), (int) g);
        run_r += pr;
        run_c += pc;
    }
    if (tid == 255) { row_offs[G] = s_row[255]; col_offs[G] = s_col[255]; }
    for (int64_t b = s_col[255] / kMxPad + tid; b < nblocks; b += 256) table[b] = make_int4(0, 0, 0, -1);
}

// column tiles one CTA walks (16384 x 8192 bf16, both directions: one tile per CTA 0.176 ms, strips of two
// 0.162 ms, of four 0.148 ms)
#ifndef PTB_MX_STRIP
#define PTB_MX_STRIP 4
#endif
constexpr int kMxStrip = PTB_MX_STRIP;
__device__ __forceinline__ void mx_cp_async16_zfill(void *dst_smem, const void *src, bool valid) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t) __cvta_generic_to_shared(dst_smem)), "l"(src),
                 "r"(valid ? 16u : 0u)
                 : "memory");
}

template <typename T> __device__ __forceinline__ void decode8(const uint4 &raw, float (&v)[8]) {
    const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = to_f32(e[i]);
}

template <int FMT> __device__ __forceinline__ uint32_t mx_cvt4(const float *v, float inv) {
    float c[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) c[i] = __fmul_rn(v[i], inv);
    return (uint32_t) cvt_fp8x2<FMT>(c[0], c[1]) | ((uint32_t) cvt_fp8x2<FMT>(c[2], c[3]) << 16);
}

// grid: (ceil(N_pad / 128 / kMxStrip), M_pad / 128, G); 256 threads; warp w: rows 32 * (w & 3), columns 64 * (w >> 2) of a tile
// GROUPED: blockIdx.y walks the 128-row blocks of the padded column layout; the block table says which
// source rows it holds and where they go in the row-direction output; a block maximum of zero takes scale
// byte 127 (1.0) instead of 0, as the reference's grouped kernel does (quantization_mxfp8.cu:1425-1450).
template <typename T, int FMT, bool GROUPED>
__global__ void __launch_bounds__(256, PTB_MXQ_MINB) mx_quant_kernel(const MxQuantArgs p) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rl = lane >> 3, cl = lane & 7;
    const int64_t g    = GROUPED ? 0 : blockIdx.z;
    const int64_t row0 = (int64_t) blockIdx.y * 128 + 32 * (warp & 3); // row of the (padded) column layout
    const T *x         = reinterpret_cast<const T *>(p.x) + g * p.M * p.N;
    int64_t src0 = row0, src_end = p.M, out0 = row0; // first source row of this warp, end of valid rows, its row-output row
    if constexpr (GROUPED) {
        const int4 e = p.table[blockIdx.y];
        src0         = (int64_t) e.x + 32 * (warp & 3);
        src_end      = e.y;
        out0         = (int64_t) e.z + 32 * (warp & 3);
    }

    // A CTA walks kMxStrip consecutive column tiles; the fragments of the tile after the current one are already
    // on their way (cp.async into this thread's own shared-memory slots, zero-filled outside the matrix).
    __shared__ uint4 s_frag[8][256];
    const int tiles_x = (int) (p.N_pad / 128);
    const int tx0     = (int) blockIdx.x * kMxStrip;
    const int ntiles  = min(kMxStrip, tiles_x - tx0);
    auto issue = [&](int t) {
        const int64_t c = (int64_t) (tx0 + t) * 128 + 64 * (warp >> 2) + cl * 8;
#pragma unroll
        for (int ps = 0; ps < 8; ++ps) {
            const int64_t r  = src0 + 4 * ps + rl;
            const bool valid = r < src_end && c < p.N;
            mx_cp_async16_zfill(&s_frag[ps][threadIdx.x], valid ? (const void *) (x + r * p.N + c) : (const void *) x, valid);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    issue(0);
    for (int t = 0; t < ntiles; ++t) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    uint4 raw[8];
#pragma unroll
    for (int ps = 0; ps < 8; ++ps) raw[ps] = s_frag[ps][threadIdx.x];
    if (t + 1 < ntiles) issue(t + 1);
    const int64_t col0 = (int64_t) (tx0 + t) * 128 + 64 * (warp >> 2);
    const int64_t col  = col0 + cl * 8;
    float rmax[8], cmax[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) cmax[j] = 0.0f;
#pragma unroll
    for (int ps = 0; ps < 8; ++ps) {
        float v[8];
        decode8<T>(raw[ps], v);
        float m = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float a = fabsf(v[j]);
            m             = fmaxf(m, a);
            cmax[j]       = fmaxf(cmax[j], a);
        }
        m        = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
        rmax[ps] = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2)); // the four lanes of a 32-column block
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        cmax[j] = fmaxf(cmax[j], __shfl_xor_sync(0xffffffffu, cmax[j], 8));
        cmax[j] = fmaxf(cmax[j], __shfl_xor_sync(0xffffffffu, cmax[j], 16)); // the four lanes that share a column
    }
    float tmax = 0.0f; // maximum of the 32x32 tile this lane's columns belong to
    if (p.row_2d || p.col_2d) {
#pragma unroll
        for (int j = 0; j < 8; ++j) tmax = fmaxf(tmax, cmax[j]);
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
    }

    // ---- row direction: q_row[g][r][col .. col+7], s_row[g][r][col / 32] -----------------------------
    if (p.q_row != nullptr) {
        uint8_t *q       = p.q_row + g * p.M * p.N_pad;
        uint8_t *s       = p.s_row + g * p.M * (p.N_pad / kMxBlock);
        const int tile_b = mx_byte<FMT, GROUPED>(tmax);
#pragma unroll
        for (int ps = 0; ps < 8; ++ps) {
            if (src0 + 4 * ps + rl >= src_end) continue; // only rows that exist are written
            const int64_t r  = out0 + 4 * ps + rl;
            const int biased = p.row_2d ? tile_b : mx_byte<FMT, GROUPED>(rmax[ps]);
            const float inv = mx_inverse(biased);
            float v[8];
            decode8<T>(raw[ps], v);
            *reinterpret_cast<uint2 *>(q + r * p.N_pad + col) = make_uint2(mx_cvt4<FMT>(v, inv), mx_cvt4<FMT>(v + 4, inv));
            if ((cl & 3) == 0) s[r * (p.N_pad / kMxBlock) + col / kMxBlock] = (uint8_t) biased;
        }
    }

    // ---- column direction: q_col[g][c][row0 .. row0+31] (transposed), s_col[g][c][row0 / 32] ---------
    if (p.q_col != nullptr) {
        uint8_t *q = p.q_col + g * p.N * p.M_pad;
        uint8_t *s = p.s_col + g * p.N * (p.M_pad / kMxBlock);
        const int tile_b = mx_byte<FMT, GROUPED>(tmax);
        // two passes of four columns each keep the live state small
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float inv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int j      = 4 * h + i;
                const int biased = p.col_2d ? tile_b : mx_byte<FMT, GROUPED>(cmax[j]);
                inv[i] = mx_inverse(biased);
                if (rl == 0 && col + j < p.N) s[(col + j) * (p.M_pad / kMxBlock) + row0 / kMxBlock] = (uint8_t) biased;
            }
            // w[ps]: this lane's row (4 ps + rl), columns 4 h .. 4 h + 3, one byte each
            uint32_t w[8];
#pragma unroll
            for (int ps = 0; ps < 8; ++ps) {
                const T *e = reinterpret_cast<const T *>(&raw[ps]) + 4 * h;
                float c[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) c[i] = __fmul_rn(to_f32(e[i]), inv[i]);
                w[ps] = (uint32_t) cvt_fp8x2<FMT>(c[0], c[1]) | ((uint32_t) cvt_fp8x2<FMT>(c[2], c[3]) << 16);
            }
            // 4x4 byte transpose across the lanes rl = 0..3 (lane bits 3 and 4): afterwards byte k of
            // w[ps] is row 4 ps + k of column 4 h + rl
#pragma unroll
            for (int ps = 0; ps < 8; ++ps) {
                uint32_t mine  = w[ps];
                uint32_t other = __shfl_xor_sync(0xffffffffu, mine, 8);
                mine           = (rl & 1) ? __byte_perm(mine, other, 0x3715) : __byte_perm(mine, other, 0x6240);
                other          = __shfl_xor_sync(0xffffffffu, mine, 16);
                mine           = (rl & 2) ? __byte_perm(mine, other, 0x3276) : __byte_perm(mine, other, 0x5410);
                w[ps]          = mine;
            }
            const int64_t c = col + 4 * h + rl;
            if (c < p.N) {
                uint4 *dst = reinterpret_cast<uint4 *>(q + c * p.M_pad + row0);
                dst[0]     = make_uint4(w[0], w[1], w[2], w[3]);
                dst[1]     = make_uint4(w[4], w[5], w[6], w[7]);
            }
        }
    }
    } // column tiles of the strip
}

// out[r][c] = cast(float(q[r][c]) * (scale byte << 23 read as fp32)); TRANSPOSE writes out[c][r] instead
template <typename TO, int FMT, bool TRANSPOSE>
__global__ void __launch_bounds__(256) mx_dequant_kernel(const uint8_t *__restrict__ q, const uint8_t *__restrict__ s,
                                                         int64_t R, int64_t C, TO *__restrict__ out) {
    __shared__ float tile[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5; // 32 x 8
    const int64_t c0 = (int64_t) blockIdx.x * 32, r0 = (int64_t) blockIdx.y * 32;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t r = r0 + ty + 8 * i, c = c0 + tx;
        float v = 0.0f;
        if (r < R && c < C) {
            const float sc = __uint_as_float((uint32_t) s[r * (C / kMxBlock) + c / kMxBlock] << 23);
            v              = __fmul_rn(fp8_to_f32<FMT>(q[r * C + c]), sc);
        }
        if constexpr (TRANSPOSE) tile[ty + 8 * i][tx] = v;
        else if (r < R && c < C) out[r * C + c] = from_f32<TO>(v);
    }
    if constexpr (TRANSPOSE) {
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int64_t c = c0 + ty + 8 * i, r = r0 + tx; // out is [C][R]
            if (r < R && c < C) out[c * R + r] = from_f32<TO>(tile[tx][ty + 8 * i]);
        }
    }
}

} // namespace
} // namespace ptb

using namespace ptb;

extern "C" {
#pragma GCC visibility push(default)

int ptb_quant_mxfp8(const void *x, int x_dtype, int64_t G, int64_t M, int64_t N, void *q_row, void *s_row,
                    void *q_col, void *s_col, int row_2d_block, int col_2d_block, int q_dtype, ptb_stream_t stream) {
    PTB_REQUIRE(x_dtype == PTB_BF16 || x_dtype == PTB_F16, PTB_ERR_ARG, "MXFP8 quantise takes bf16 or fp16 input, got dtype %d", x_dtype);
    PTB_REQUIRE(is_fp8(q_dtype), PTB_ERR_ARG, "MXFP8 quantise output must be e4m3 or e5m2, got dtype %d", q_dtype);
    PTB_REQUIRE(G >= 0 && M >= 0 && N >= 0, PTB_ERR_ARG, "negative extent");
    PTB_REQUIRE(N % kMxBlock == 0, PTB_ERR_ARG, "N (%lld) must be divisible by 32", (long long) N);
    PTB_REQUIRE((q_row == nullptr) == (s_row == nullptr) && (q_col == nullptr) == (s_col == nullptr), PTB_ERR_ARG,
                "each direction needs both its data and its scale output");
    PTB_REQUIRE(q_row != nullptr || q_col != nullptr, PTB_ERR_ARG, "no output requested");
    if (G == 0 || M == 0 || N == 0) return 0;
    PTB_REQUIRE(aligned16(x) && (q_row == nullptr || aligned16(q_row)) && (q_col == nullptr || aligned16(q_col)), PTB_ERR_ARG,
                "MXFP8 quantise needs 16-byte aligned input and FP8 outputs");
    MxQuantArgs a;
    a.x = x; a.q_row = (uint8_t *) q_row; a.s_row = (uint8_t *) s_row; a.q_col = (uint8_t *) q_col; a.s_col = (uint8_t *) s_col;
    a.M = M; a.N = N; a.M_pad = cdiv<int64_t>(M, kMxPad) * kMxPad; a.N_pad = cdiv<int64_t>(N, kMxPad) * kMxPad;
    a.row_2d = row_2d_block; a.col_2d = col_2d_block;
    PTB_REQUIRE(a.M_pad / 128 <= 65535 && G <= 65535, PTB_ERR_ARG, "MXFP8 quantise: more than 65535 row tiles or groups");
    dim3 grid((unsigned) cdiv<int64_t>(a.N_pad / 128, kMxStrip), (unsigned) (a.M_pad / 128), (unsigned) G);
    cudaStream_t st = (cudaStream_t) stream;
    a.table = nullptr;
    if (x_dtype == PTB_BF16) {
        PTB_SWITCH_FP8(q_dtype, FMT, (mx_quant_kernel<__nv_bfloat16, FMT, false><<<grid, 256, 0, st>>>(a)));
    } else {
        PTB_SWITCH_FP8(q_dtype, FMT, (mx_quant_kernel<__half, FMT, false><<<grid, 256, 0, st>>>(a)));
    }
    PTB_LAUNCH_CHECK("mx_quant_kernel");
    return 0;
}

int ptb_quant_mxfp8_grouped(const void *x, int x_dtype, int64_t M, int64_t N, const int64_t *group_offs, int64_t G,
                            int64_t row_align, void *q_row, void *s_row, void *q_col, void *s_col, int64_t *row_lens_padded,
                            int64_t *row_offs_padded, int64_t *col_lens_padded, int64_t *col_offs_padded, void *block_table,
                            int row_2d_block, int col_2d_block, int q_dtype, ptb_stream_t stream) {
    PTB_REQUIRE(x_dtype == PTB_BF16 || x_dtype == PTB_F16, PTB_ERR_ARG, "MXFP8 quantise takes bf16 or fp16 input, got dtype %d", x_dtype);
    PTB_REQUIRE(is_fp8(q_dtype), PTB_ERR_ARG, "MXFP8 quantise output must be e4m3 or e5m2, got dtype %d", q_dtype);
    PTB_REQUIRE(G >= 1 && M >= 0 && N >= 0, PTB_ERR_ARG, "grouped MXFP8 quantise: at least one group, non-negative extents");
    PTB_REQUIRE(N % kMxBlock == 0, PTB_ERR_ARG, "N (%lld) must be divisible by 32", (long long) N);
    PTB_REQUIRE(row_align == 1 || row_align == 32, PTB_ERR_ARG, "row_align must be 1 or 32");
    // with no row at all (an expert-parallel rank that received nothing) x and an unpadded row copy are empty
    PTB_REQUIRE(group_offs && (M == 0 || (q_row && s_row)) && q_col && s_col && row_lens_padded && row_offs_padded &&
                    col_lens_padded && col_offs_padded && block_table,
                PTB_ERR_ARG, "grouped MXFP8 quantise: null pointer");
    PTB_REQUIRE(M < (1ll << 31), PTB_ERR_TOO_LARGE, "grouped MXFP8 quantise: too many rows");
    PTB_REQUIRE((N == 0 || aligned16(x)) && aligned16(q_row) && aligned16(q_col) && aligned16(block_table), PTB_ERR_ARG,
                "MXFP8 quantise needs 16-byte aligned input, FP8 outputs and block table");
    MxQuantArgs a;
    a.x = x ? x : q_col; // never dereferenced without rows; the zero-size copies still get a mapped address
    a.q_row = (uint8_t *) q_row; a.s_row = (uint8_t *) s_row; a.q_col = (uint8_t *) q_col; a.s_col = (uint8_t *) s_col;
    a.M = M; a.N = N;
    a.M_pad = cdiv<int64_t>(M + G * kMxPad, kMxPad) * kMxPad; // rows the column layout is allocated for (upper bound)
    a.N_pad = cdiv<int64_t>(N, kMxPad) * kMxPad;
    a.row_2d = row_2d_block; a.col_2d = col_2d_block;
    a.table  = (const int4 *) block_table;
    const int64_t nblocks = a.M_pad / kMxPad;
    PTB_REQUIRE(nblocks <= 65535, PTB_ERR_TOO_LARGE, "grouped MXFP8 quantise: more than 65535 row blocks");
    cudaStream_t st = (cudaStream_t) stream;
    mx_group_layout_kernel<<<1, 256, 0, st>>>(group_offs, G, row_align, row_lens_padded, row_offs_padded, col_lens_padded,
                                              col_offs_padded, (int4 *) block_table, nblocks);
    PTB_LAUNCH_CHECK("mx_group_layout_kernel");
    if (N == 0) return 0;
    dim3 grid((unsigned) cdiv<int64_t>(a.N_pad / 128, kMxStrip), (unsigned) nblocks, 1);
    if (x_dtype == PTB_BF16) {
        PTB_SWITCH_FP8(q_dtype, FMT, (mx_quant_kernel<__nv_bfloat16, FMT, true><<<grid, 256, 0, st>>>(a)));
    } else {
        PTB_SWITCH_FP8(q_dtype, FMT, (mx_quant_kernel<__half, FMT, true><<<grid, 256, 0, st>>>(a)));
    }
    PTB_LAUNCH_CHECK("mx_quant_kernel");
    return 0;
}

int ptb_dequant_mxfp8(const void *q, int q_dtype, int64_t R, int64_t C, const void *scales, int transpose_out, void *out,
                      int out_dtype, ptb_stream_t stream) {
    PTB_REQUIRE(is_fp8(q_dtype) && is_hp(out_dtype), PTB_ERR_ARG, "MXFP8 dequantise: unsupported dtypes %d -> %d", q_dtype, out_dtype);
    PTB_REQUIRE(R >= 0 && C >= 0 && C % kMxBlock == 0, PTB_ERR_ARG, "MXFP8 dequantise: the inner extent (%lld) must be divisible by 32", (long long) C);
    if (R == 0 || C == 0) return 0;
    PTB_REQUIRE(cdiv<int64_t>(R, 32) <= 65535, PTB_ERR_ARG, "MXFP8 dequantise: more than 65535 row tiles");
    dim3 grid((unsigned) cdiv<int64_t>(C, 32), (unsigned) cdiv<int64_t>(R, 32));
    cudaStream_t st = (cudaStream_t) stream;
    const uint8_t *qq = (const uint8_t *) q, *ss = (const uint8_t *) scales;
#define PTB_MX_DQ(TO)                                                                                          \
    if (transpose_out) { PTB_SWITCH_FP8(q_dtype, FMT, (mx_dequant_kernel<TO, FMT, true><<<grid, 256, 0, st>>>(qq, ss, R, C, (TO *) out))); } \
    else { PTB_SWITCH_FP8(q_dtype, FMT, (mx_dequant_kernel<TO, FMT, false><<<grid, 256, 0, st>>>(qq, ss, R, C, (TO *) out))); }
    if (out_dtype == PTB_BF16) { PTB_MX_DQ(__nv_bfloat16) }
    else if (out_dtype == PTB_F16) { PTB_MX_DQ(__half) }
    else { PTB_MX_DQ(float) }
#undef PTB_MX_DQ
    PTB_LAUNCH_CHECK("mx_dequant_kernel");
    return 0;
}

#pragma GCC visibility pop
}
