// Variable-K grouped GEMM with 1-D x 1-D block scales (the blockwise wgrad), paired-tile form.
// Included by ptb_gemm.cu (it uses that file's PTX wrappers, tensor-map helpers and status word).
//
// Why a second kernel.  In wgrad every output tile sees only two or three 128-row contraction blocks,
// and each block's partial product must be multiplied by a row scale AND a column scale before it is
// added up.  A thread owns one TMEM lane (= one output row), so the row scale is one register, but the
// column scales are a different value for every column it holds, re-read from shared memory for every
// block: with a 128 x 256 tile that is 128 KiB of broadcast reads per block and CTA, as much as the
// partial product itself, and the shared-memory pipe (also fed by the TMA writes, the tensor cores'
// operand reads and the output staging) is what the general kernel saturates.
// Here a tile is 256 rows x 128 columns, computed as TWO 128 x 128 products that share the B tile and
// land side by side in one 256-column TMEM buffer.  A thread now holds the same 64 columns of two
// rows, so every column scale it fetches serves two elements: half the broadcast traffic for the
// same tile area, the same TMEM loads, the same arithmetic, the same output staging.
//
// One persistent CTA per SM, 384 threads:
//   warp 0      TMA producer: 3-stage ring of {A0 16 KiB, A1 16 KiB, B 16 KiB}, all MN-major.
//   warp 1      MMA issuer: per stage 2 x 4 tcgen05.mma (M128 N128 K32), accumulate flag cleared per block.
//   warp 2      TMEM allocation.
//   warp 3      scale loader: 256 row scales + 128 column scales per block into a 4-slot ring (cp.async).
//   warps 4-11  promotion + epilogue: quadrant = warp & 3 (TMEM lanes), half = 64-column slice.
// Requirements (checked by the launcher, which otherwise uses the general kernel): OUT_M % 256 == 0,
// OUT_N % 128 == 0, 16-bit output reachable by TMA stores, every group offset a multiple of 128.
#pragma once

namespace ptb {
namespace {

constexpr int kWgStages     = 3;
constexpr int kWgStageBytes = 3 * 16384;
constexpr int kWgCStage     = 8 * 2 * 4096; // eight warps x two 32-row x 64-column slabs of 16-bit values
constexpr int kWgSlotFloats = 256 + 128;
constexpr int kWgThreads    = 384;

struct __align__(16) WgCtl {
    float scale_ring[kScaleSlots * kWgSlotFloats];
    uint64_t sc_full[kScaleSlots];
    uint64_t sc_empty[kScaleSlots];
    uint64_t full[kWgStages];
    uint64_t empty[kWgStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    int group_offs[kMaxGroups + 1];
};

struct WgTile {
    int m0, n0, g, k_row0, num_kb;
};

// tiles blockIdx.x, blockIdx.x + gridDim.x, ... in (group, row pair, column tile) order, column tiles fastest;
// the grid stride is split into its three digits once, later tiles are reached by addition and carry
struct WgSchedule {
    int g, pm, nt;       // current tile
    int sg, spm, snt;    // grid stride, split
    int pairs_m, tiles_n, G;
    const int *offs;
    __device__ WgSchedule(const GemmArgs &a, const WgCtl *ctl) {
        pairs_m = a.M / 256; tiles_n = a.N / 128; G = a.G; offs = ctl->group_offs;
        const int per_g = pairs_m * tiles_n;
        int lin = blockIdx.x;
        g = lin / per_g; lin -= g * per_g; pm = lin / tiles_n; nt = lin - pm * tiles_n;
        int st = gridDim.x;
        sg = st / per_g; st -= sg * per_g; spm = st / tiles_n; snt = st - spm * tiles_n;
    }
    __device__ bool get(WgTile &t) {
        if (g >= G) return false;
        const int lo = offs[g], hi = offs[g + 1];
        t.m0 = pm * 256; t.n0 = nt * 128; t.g = g; t.k_row0 = lo; t.num_kb = (hi - lo) / BK;
        nt += snt; pm += spm; g += sg;
        if (nt >= tiles_n) { nt -= tiles_n; ++pm; }
        if (pm >= pairs_m) { pm -= pairs_m; ++g; }
        return true;
    }
};

// 16-byte global -> shared copy that occupies no register while in flight
__device__ __forceinline__ void cp_async_16(float *dst_smem, const float *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}

template <typename OutT>
__global__ void __launch_bounds__(kWgThreads, 1) wgrad_pair_kernel(const __grid_constant__ GemmArgs args) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem    = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *c_stage = smem + kWgStages * kWgStageBytes;
    WgCtl *ctl       = reinterpret_cast<WgCtl *>(c_stage + kWgCStage);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem_base = smem_u32(smem);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kWgStages; ++s) {
            mbar_init(smem_u32(&ctl->full[s]), 1);
            mbar_init(smem_u32(&ctl->empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&ctl->tmem_full[b]), 1);
            mbar_init(smem_u32(&ctl->tmem_empty[b]), 8); // one arrival per promotion warp
        }
        for (int b = 0; b < kScaleSlots; ++b) {
            mbar_init(smem_u32(&ctl->sc_full[b]), 32);
            mbar_init(smem_u32(&ctl->sc_empty[b]), 8);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (threadIdx.x == 64) {
        tma_prefetch_map(&args.tm_a);
        tma_prefetch_map(&args.tm_b);
        tma_prefetch_map(&args.tm_c);
    }
    for (int g = threadIdx.x; g <= args.G; g += kWgThreads) ctl->group_offs[g] = (int) args.group_offs[g];
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&ctl->tmem_base))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;

    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        if (warp == 0 && lane == 0) {
            // ================= TMA producer =================
            WgSchedule sched(args, ctl);
            WgTile t;
            uint32_t it = 0;
            bool ok     = true;
            while (ok && sched.get(t)) {
                for (int kb = 0; kb < t.num_kb; ++kb, ++it) {
                    const int s = it % kWgStages;
                    if (!mbar_wait(smem_u32(&ctl->empty[s]), ((it / kWgStages) & 1) ^ 1)) { ok = false; break; }
                    const uint32_t full = smem_u32(&ctl->full[s]);
                    mbar_expect_tx(full, kWgStageBytes);
                    const uint32_t sa = smem_base + s * kWgStageBytes;
                    const int k = t.k_row0 + kb * BK;
                    tma_load_3d(sa, &args.tm_a, full, t.m0, k, 0);
                    tma_load_3d(sa + 16384, &args.tm_a, full, t.m0 + 128, k, 0);
                    tma_load_3d(sa + 32768, &args.tm_b, full, t.n0, k, 0);
                }
            }
            if (!ok) {
                atomicExch(&g_gemm_status, 1);
                const uint32_t back = it < (uint32_t) kWgStages ? it : (uint32_t) kWgStages;
                for (uint32_t j = 1; j <= back; ++j) {
                    const uint32_t q = it - j;
                    mbar_wait(smem_u32(&ctl->full[q % kWgStages]), (q / kWgStages) & 1);
                }
            }
        } else if (warp == 1) {
            // ================= MMA issuer =================
            WgSchedule sched(args, ctl);
            WgTile t;
            uint32_t it = 0;
            bool ok     = true;
            while (ok && sched.get(t)) {
                for (int kb = 0; kb < t.num_kb; ++kb, ++it) {
                    const int s = it % kWgStages;
                    const uint32_t buf = it & 1;
                    if (!mbar_wait(smem_u32(&ctl->tmem_empty[buf]), ((it >> 1) & 1) ^ 1)) { ok = false; break; }
                    if (!mbar_wait(smem_u32(&ctl->full[s]), (it / kWgStages) & 1)) { ok = false; break; }
                    tc_fence_after();
                    if (lane == 0) {
                        const uint32_t sa = smem_base + s * kWgStageBytes;
                        const uint64_t a0 = make_smem_desc(sa, 0, 1024), a1 = make_smem_desc(sa + 16384, 0, 1024);
                        const uint64_t bd = make_smem_desc(sa + 32768, 0, 1024);
                        const uint32_t d  = tmem_base + buf * 256;
#pragma unroll
                        for (int j = 0; j < BK / 32; ++j) // 32 contraction rows of an MN-major tile = 4096 bytes
                            tc_mma_f8(d, a0 + (uint64_t) ((4096u * j) >> 4), bd + (uint64_t) ((4096u * j) >> 4), args.idesc, j > 0);
#pragma unroll
                        for (int j = 0; j < BK / 32; ++j)
                            tc_mma_f8(d + 128, a1 + (uint64_t) ((4096u * j) >> 4), bd + (uint64_t) ((4096u * j) >> 4), args.idesc,
                                      j > 0);
                        tc_commit(smem_u32(&ctl->empty[s]));
                        tc_commit(smem_u32(&ctl->tmem_full[buf]));
                    }
                    __syncwarp();
                }
            }
            if (!ok && lane == 0) atomicExch(&g_gemm_status, 2);
        } else if (warp == 3) {
            // ================= scale loader =================
            WgSchedule sched(args, ctl);
            WgTile t;
            uint32_t it = 0;
            bool ok     = true;
            while (ok && sched.get(t)) {
                const int kb_base = t.k_row0 / BK;
                for (int kb = 0; kb < t.num_kb; ++kb, ++it) {
                    const int slot = it % kScaleSlots;
                    if (!mbar_wait(smem_u32(&ctl->sc_empty[slot]), ((it / kScaleSlots) & 1) ^ 1)) { ok = false; break; }
                    float *dst         = &ctl->scale_ring[slot * kWgSlotFloats];
                    const float *a_src = args.a_scale + (int64_t) (kb_base + kb) * args.as_k + t.m0; // 256 contiguous floats
                    const float *b_src = args.b_scale + (int64_t) (kb_base + kb) * args.bs_k + t.n0; // 128 contiguous floats
                    cp_async_16(dst + lane * 4, a_src + lane * 4);
                    cp_async_16(dst + 128 + lane * 4, a_src + 128 + lane * 4);
                    cp_async_16(dst + 256 + lane * 4, b_src + lane * 4);
                    cp_async_arrive_on(smem_u32(&ctl->sc_full[slot]));
                }
            }
            cp_async_wait_all();
            if (!ok && lane == 0) atomicExch(&g_gemm_status, 4);
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
        // ================= promotion + epilogue =================
        const int half = (warp - 4) >> 2; // 64-column slice
        const int quad = warp & 3;        // TMEM lane quadrant
        const int row_in_tile = quad * 32 + lane;
        uint8_t *my_stage        = c_stage + (warp - 4) * 8192;
        const uint32_t stage_u32 = smem_u32(my_stage);
        WgSchedule sched(args, ctl);
        WgTile t;
        uint32_t it        = 0;
        bool ok            = true;
        bool store_pending = false;
        float acc[128]; // [0, 64): row of the first 128-row tile, [64, 128): same lane's row of the second
        while (ok && sched.get(t)) {
#pragma unroll
            for (int j = 0; j < 128; ++j) acc[j] = 0.0f;
            for (int kb = 0; kb < t.num_kb; ++kb, ++it) {
                const uint32_t buf = it & 1;
                const int slot     = it % kScaleSlots;
                if (!mbar_wait(smem_u32(&ctl->sc_full[slot]), (it / kScaleSlots) & 1)) { ok = false; break; }
                const float *sl = &ctl->scale_ring[slot * kWgSlotFloats];
                const float r0 = sl[row_in_tile], r1 = sl[128 + row_in_tile];
                const float2 r0v = make_float2(r0, r0), r1v = make_float2(r1, r1);
                const float *cs = sl + 256 + half * 64;
                if (!mbar_wait(smem_u32(&ctl->tmem_full[buf]), (it >> 1) & 1)) { ok = false; break; }
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t) (quad * 32) << 16) + buf * 256 + half * 64;
                float va[16], vb[16], vc[16], vd[16];
                tc_ld16(taddr, va);
                tc_ld16(taddr + 128, vb);
                tc_wait_ld();
// one 16-column chunk of both rows: every column scale read serves two elements
#define PTB_WG_PROMOTE(V0, V1, C)                                                                             \
    _Pragma("unroll") for (int j = 0; j < 4; ++j) {                                                           \
        const float4 c4 = *reinterpret_cast<const float4 *>(cs + (C) * 16 + 4 * j);                           \
        const float2 cl = make_float2(c4.x, c4.y), ch = make_float2(c4.z, c4.w);                              \
        float2 a;                                                                                             \
        a = __ffma2_rn(__fmul2_rn(make_float2(V0[4 * j], V0[4 * j + 1]), r0v), cl,                            \
                       make_float2(acc[(C) * 16 + 4 * j], acc[(C) * 16 + 4 * j + 1]));                        \
        acc[(C) * 16 + 4 * j] = a.x; acc[(C) * 16 + 4 * j + 1] = a.y;                                         \
        a = __ffma2_rn(__fmul2_rn(make_float2(V0[4 * j + 2], V0[4 * j + 3]), r0v), ch,                        \
                       make_float2(acc[(C) * 16 + 4 * j + 2], acc[(C) * 16 + 4 * j + 3]));                    \
        acc[(C) * 16 + 4 * j + 2] = a.x; acc[(C) * 16 + 4 * j + 3] = a.y;                                     \
        a = __ffma2_rn(__fmul2_rn(make_float2(V1[4 * j], V1[4 * j + 1]), r1v), cl,                            \
                       make_float2(acc[64 + (C) * 16 + 4 * j], acc[64 + (C) * 16 + 4 * j + 1]));              \
        acc[64 + (C) * 16 + 4 * j] = a.x; acc[64 + (C) * 16 + 4 * j + 1] = a.y;                               \
        a = __ffma2_rn(__fmul2_rn(make_float2(V1[4 * j + 2], V1[4 * j + 3]), r1v), ch,                        \
                       make_float2(acc[64 + (C) * 16 + 4 * j + 2], acc[64 + (C) * 16 + 4 * j + 3]));          \
        acc[64 + (C) * 16 + 4 * j + 2] = a.x; acc[64 + (C) * 16 + 4 * j + 3] = a.y;                           \
    }
                tc_ld16(taddr + 16, vc);
                tc_ld16(taddr + 128 + 16, vd);
                PTB_WG_PROMOTE(va, vb, 0)
                tc_wait_ld();
                tc_ld16(taddr + 32, va);
                tc_ld16(taddr + 128 + 32, vb);
                PTB_WG_PROMOTE(vc, vd, 1)
                tc_wait_ld();
                tc_ld16(taddr + 48, vc);
                tc_ld16(taddr + 128 + 48, vd);
                PTB_WG_PROMOTE(va, vb, 2)
                tc_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ctl->tmem_empty[buf])); // the whole partial is in registers
                PTB_WG_PROMOTE(vc, vd, 3)
#undef PTB_WG_PROMOTE
                __syncwarp(); // every lane has read its scales: the loader may refill the slot
                if (lane == 0) mbar_arrive(smem_u32(&ctl->sc_empty[slot]));
            }
            if (!ok) break;
            // ---- convert, stage (128-byte swizzled), TMA store: two 32-row x 64-column slabs per warp ----
            if (store_pending) {
                if (lane == 0) tma_store_wait_read();
                __syncwarp();
            }
#pragma unroll
            for (int j8 = 0; j8 < 16; ++j8) {
                const uint32_t dst = stage_u32 + (j8 >> 3) * 4096 + lane * 128 + (((j8 & 7) ^ (lane & 7)) << 4);
                st_shared_v4(dst, Pack8<OutT>::pack(&acc[j8 * 8]));
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                const int col0 = t.n0 + half * 64, row0 = t.m0 + quad * 32;
                tma_store_3d(&args.tm_c, stage_u32, col0, row0, t.g);
                tma_store_3d(&args.tm_c, stage_u32 + 4096, col0, row0 + 128, t.g);
                tma_store_commit();
            }
            store_pending = true;
        }
        if (store_pending && lane == 0) tma_store_wait_all();
        if (!ok && lane == 0) atomicExch(&g_gemm_status, 3);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
}

constexpr size_t kWgSmemBytes = 1024 + (size_t) kWgStages * kWgStageBytes + kWgCStage + sizeof(WgCtl);
static_assert(kWgSmemBytes <= 232448, "shared memory budget of one CTA exceeded");

template <typename OutT> int launch_wgrad_pair(const GemmArgs &args, int grid, cudaStream_t st) {
    static bool configured[64] = {};
    auto kfn = wgrad_pair_kernel<OutT>;
    int dev  = 0;
    PTB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        PTB_CUDA(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) kWgSmemBytes));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    kfn<<<grid, kWgThreads, kWgSmemBytes, st>>>(args);
    PTB_LAUNCH_CHECK("wgrad_pair_kernel");
    return 0;
}

} // namespace
} // namespace ptb
