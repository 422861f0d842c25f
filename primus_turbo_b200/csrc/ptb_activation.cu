// SwiGLU with routing probabilities (the activation between the gate+up and down projections of an MoE
// expert): out[t, j] = silu(x[t, j]) * x[t, H + j] * probs[t], and its backward pass.  HBM-bound
// elementwise kernels: 16-byte accesses, fp32 arithmetic, one rounding to the storage type at the end.
// The same `swiglu_prob` device function feeds the fused quantiser in ptb_quant.cu, so
// quantise(swiglu(x)) and the fused kernel produce identical bytes.
#include "ptb_common.cuh"

namespace ptb {
namespace {

template <typename T>
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const T *__restrict__ x, const float *__restrict__ probs,
                                                          const int64_t *__restrict__ row_mask, int64_t rows, int64_t H,
                                                          T *__restrict__ out) {
    const int64_t vec_per_row = H / 8;
    const int64_t total       = rows * vec_per_row;
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t) gridDim.x * blockDim.x) {
        const int64_t r = i / vec_per_row, c = (i - r * vec_per_row) * 8;
        uint4 o         = make_uint4(0, 0, 0, 0);
        if (row_mask == nullptr || row_mask[r] != 0) {
            const uint4 u = *reinterpret_cast<const uint4 *>(x + r * 2 * H + c);
            const uint4 d = *reinterpret_cast<const uint4 *>(x + r * 2 * H + H + c);
            const T *ue = reinterpret_cast<const T *>(&u), *de = reinterpret_cast<const T *>(&d);
            T *oe         = reinterpret_cast<T *>(&o);
            const float p = probs[r];
#pragma unroll
            for (int k = 0; k < 8; ++k) oe[k] = from_f32<T>(swiglu_prob(to_f32(ue[k]), to_f32(de[k]), p));
        }
        *reinterpret_cast<uint4 *>(out + r * H + c) = o;
    }
}

// one CTA per row: grad_x[:, :H] = g*p * down * dsilu(up), grad_x[:, H:] = g*p * silu(up),
// grad_probs = sum_j g * silu(up) * down   (primus_turbo/triton/activation/swiglu_kernel.py:196-247)
template <typename T>
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const T *__restrict__ grad_out, const T *__restrict__ x,
                                                          const float *__restrict__ probs,
                                                          const int64_t *__restrict__ row_mask, int64_t rows, int64_t H,
                                                          T *__restrict__ grad_x, float *__restrict__ grad_probs) {
    __shared__ float s_red[8];
    const int64_t r = blockIdx.x;
    const bool live = row_mask == nullptr || row_mask[r] != 0;
    const float p   = probs[r];
    float sum       = 0.0f;
    for (int64_t c = (int64_t) threadIdx.x * 8; c < H; c += 256 * 8) {
        uint4 gu = make_uint4(0, 0, 0, 0), gd = make_uint4(0, 0, 0, 0);
        if (live) {
            const uint4 u = *reinterpret_cast<const uint4 *>(x + r * 2 * H + c);
            const uint4 d = *reinterpret_cast<const uint4 *>(x + r * 2 * H + H + c);
            const uint4 g = *reinterpret_cast<const uint4 *>(grad_out + r * H + c);
            const T *ue = reinterpret_cast<const T *>(&u), *de = reinterpret_cast<const T *>(&d);
            const T *ge = reinterpret_cast<const T *>(&g);
            T *gue = reinterpret_cast<T *>(&gu), *gde = reinterpret_cast<T *>(&gd);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float up = to_f32(ue[k]), down = to_f32(de[k]), go = to_f32(ge[k]);
                const float sig  = __fdiv_rn(1.0f, 1.0f + expf(-up));
                const float silu = sig * up;
                sum += go * silu * down;
                const float gop = go * p;
                gde[k]          = from_f32<T>(gop * silu);
                gue[k]          = from_f32<T>(gop * (down * (sig * (1.0f + up * (1.0f - sig)))));
            }
        }
        *reinterpret_cast<uint4 *>(grad_x + r * 2 * H + c)     = gu;
        *reinterpret_cast<uint4 *>(grad_x + r * 2 * H + H + c) = gd;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k) t += s_red[k];
        grad_probs[r] = t;
    }
}

} // namespace
} // namespace ptb

using namespace ptb;

extern "C" {
#pragma GCC visibility push(default)

int ptb_swiglu_probs_fwd(const void *x, int dtype, const float *probs, const int64_t *row_mask, int64_t rows, int64_t H,
                         void *out, ptb_stream_t stream) {
    PTB_REQUIRE(rows >= 0 && H >= 0, PTB_ERR_ARG, "swiglu_probs_fwd: negative size");
    PTB_REQUIRE(dtype == PTB_BF16 || dtype == PTB_F16, PTB_ERR_ARG, "swiglu_probs_fwd: x must be bf16 or fp16");
    PTB_REQUIRE(H % 8 == 0, PTB_ERR_ALIGN, "swiglu_probs_fwd: the hidden size must be a multiple of 8");
    if (rows == 0 || H == 0) return 0;
    PTB_REQUIRE(x && probs && out, PTB_ERR_ARG, "swiglu_probs_fwd: null pointer");
    PTB_REQUIRE(aligned16(x) && aligned16(out), PTB_ERR_ALIGN, "swiglu_probs_fwd: buffers must be 16-byte aligned");
    const int blocks = (int) imin(cdiv<int64_t>(rows * (H / 8), 256), 148 * 16);
    if (dtype == PTB_BF16)
        swiglu_fwd_kernel<__nv_bfloat16><<<blocks, 256, 0, (cudaStream_t) stream>>>((const __nv_bfloat16 *) x, probs, row_mask, rows, H, (__nv_bfloat16 *) out);
    else
        swiglu_fwd_kernel<__half><<<blocks, 256, 0, (cudaStream_t) stream>>>((const __half *) x, probs, row_mask, rows, H, (__half *) out);
    PTB_LAUNCH_CHECK("swiglu_fwd_kernel");
    return 0;
}

int ptb_swiglu_probs_bwd(const void *grad_out, const void *x, int dtype, const float *probs, const int64_t *row_mask,
                         int64_t rows, int64_t H, void *grad_x, float *grad_probs, ptb_stream_t stream) {
    PTB_REQUIRE(rows >= 0 && H >= 0, PTB_ERR_ARG, "swiglu_probs_bwd: negative size");
    PTB_REQUIRE(dtype == PTB_BF16 || dtype == PTB_F16, PTB_ERR_ARG, "swiglu_probs_bwd: x must be bf16 or fp16");
    PTB_REQUIRE(H % 8 == 0, PTB_ERR_ALIGN, "swiglu_probs_bwd: the hidden size must be a multiple of 8");
    PTB_REQUIRE(rows <= 2147483647LL, PTB_ERR_TOO_LARGE, "swiglu_probs_bwd: too many rows");
    if (rows == 0) return 0;
    PTB_REQUIRE(grad_probs && probs, PTB_ERR_ARG, "swiglu_probs_bwd: null pointer");
    PTB_REQUIRE(H == 0 || (grad_out && x && grad_x), PTB_ERR_ARG, "swiglu_probs_bwd: null pointer");
    PTB_REQUIRE(aligned16(x) && aligned16(grad_out) && aligned16(grad_x), PTB_ERR_ALIGN,
                "swiglu_probs_bwd: buffers must be 16-byte aligned");
    if (dtype == PTB_BF16)
        swiglu_bwd_kernel<__nv_bfloat16><<<(unsigned) rows, 256, 0, (cudaStream_t) stream>>>(
            (const __nv_bfloat16 *) grad_out, (const __nv_bfloat16 *) x, probs, row_mask, rows, H, (__nv_bfloat16 *) grad_x, grad_probs);
    else
        swiglu_bwd_kernel<__half><<<(unsigned) rows, 256, 0, (cudaStream_t) stream>>>(
            (const __half *) grad_out, (const __half *) x, probs, row_mask, rows, H, (__half *) grad_x, grad_probs);
    PTB_LAUNCH_CHECK("swiglu_bwd_kernel");
    return 0;
}

#pragma GCC visibility pop
} // extern "C"
