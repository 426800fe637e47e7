// fp32 ConvBias / MatrixMul on the sm_100a tensor cores with fp32-level accuracy.
//
// tcgen05.mma kind::tf32 keeps 10 mantissa bits of each operand, which is not enough for the
// 1e-4 relative tolerance the fp32 path is held to (a single tf32 pass is off by ~5e-4 on
// N(0,1) data). Every operand is therefore split into two tf32 values,
//     v = hi + lo,   hi = RN_tf32(v),   lo = RN_tf32(v - hi)          (v - hi is exact)
// and the product is accumulated in the fp32 TMEM accumulator from three passes
//     hi*hi + lo*hi + hi*lo                                            (lo*lo is < 2^-22)
// which leaves a relative error of a few 2^-22 per product: the same order as fp32 itself.
// Both halves are exactly representable in tf32, so the result does not depend on how the
// tensor core treats the low 13 bits of its inputs.
//
// The tensor core adds each MMA's products into the TMEM accumulator with truncation, not
// round-to-nearest: every instruction pulls the running sum toward zero by about half an ulp.
// Over a long chain that is a SYSTEMATIC shrink of the result (measured: K = 1152 in one
// chain scaled outputs by 1 - 4e-6; through the 60 ConvBias layers between a detector's input
// and its heads that compounded to -3.6e-4, against a tolerance of 1e-4). Two measures keep
// the drift at the level of fp32 rounding:
//   * short chains: the K loop is cut into segments of eight K = 8 steps (with four the worst
//     error of a detector's heads is 0.15 of the tolerance and the kernel 10 % slower, with
//     sixteen 0.35, with thirty-two 0.6; eight leaves 0.23); every segment starts
//     fresh TMEM accumulators (two sets alternate) and the epilogue warps add the finished
//     segment into fp32 registers with round-to-nearest while the tensor core works on the
//     next one. A short partial sum is small against the final one and nearly uncorrelated
//     with its sign, so what is left of the drift largely cancels;
//   * the two correction passes (lo*hi, hi*lo) go to an accumulator of their own: they are
//     2^-11 of the main pass, so their truncation does not matter, and they no longer cause
//     two extra truncations of the main sum per step.
//
//   * filter: split once at load time (the Init step) into two K-major planes
//     [2][OC][KH][KW][IC];
//   * activation: fetched as it is by TMA (im2col, or tiled for a 1x1 filter) and split ON
//     CHIP: four converter warps turn each arrived fp32 tile into its hi plane in place and
//     its lo plane in the neighbouring slot of the stage. The split is elementwise and the
//     TMA swizzle is a function of the shared-memory address, so both planes keep the layout
//     the MMA descriptors expect; no pre-pass over global memory, no scratch tensor, and the
//     input is read once instead of five times (read, two plane writes, two plane reads);
//   * structure of the kernel as in conv_umma.cu: persistent CTAs, warp 0 TMA producer, warp 1
//     MMA issuer and TMEM owner, warps 2..9 epilogue (tcgen05.ld -> + bias -> activation ->
//     optional residual add -> 16-byte NHWC stores), warps 10..13 converters, two accumulator
//     buffers, bounded waits.
//
// Replaces, for the fp32 configurations, the reference's im2col + 4x12 SIMD GEMM
// (compiler/lib/KernelGen/GeneralIntrinsic/ConvKernel/Fp32Im2col.cpp:122-217,
// GeneralIntrinsic/MatMulKernel/Fp32MatMulM4N12.cpp:8-160) and the SILU / SIGMOID elementwise
// kernel that follows a ConvBias in a YOLOX-style graph
// (BareMetal/ElemwiseKernel.cpp:52-53, BareMetal/Activation.cpp:31-37). Summation order
// differs from the reference's, as it does between any two fp32 GEMMs: parity is held to
// 1e-4 relative / 1e-5 absolute, not bit for bit.
#include <stdio.h>
#include <stdlib.h>

#include "f32_internal.h"
#include "pdl.h"
#include "tuning.h"
#include "umma_ptx.cuh"

namespace mb200 {

using namespace umma;

namespace {

constexpr int kBM = 128;
constexpr int kMaxStages = 6;

// kind::tf32 instruction descriptor: fp32 accumulate, tf32 A and B, both K-major
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int m, int n) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

template <bool ACCUMULATE>
__device__ __forceinline__ void umma_tf32_c(
        uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
    asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "n"(ACCUMULATE ? 1 : 0)
            : "memory");
}

__device__ __forceinline__ void umma_tf32(
        uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
}

// round to the nearest tf32 (ties to even): keeps sign, 8 exponent and 10 mantissa bits
__host__ __device__ inline float round_tf32(float v) {
    uint32_t u;
    memcpy(&u, &v, 4);
    u = (u + 0xFFFu + ((u >> 13) & 1u)) & 0xFFFFE000u;
    float r;
    memcpy(&r, &u, 4);
    return r;
}

// ------------------------------------------------------------------------------------------
// filter packing (load time)
// ------------------------------------------------------------------------------------------
// OIHW fp32 -> two K-major planes [2][OC][KH][KW][ICp] (hi, lo), ICp >= IC zero-filled
__global__ void __launch_bounds__(256) pack_filter_f32_kernel(
        const float* __restrict__ src, float* __restrict__ dst, int oc, int ic, int icp, int kh,
        int kw) {
    const size_t plane = (size_t)oc * kh * kw * icp;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < plane;
         i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % icp);
        size_t t = i / icp;
        const int fx = (int)(t % kw);
        t /= kw;
        const int fy = (int)(t % kh);
        const int o = (int)(t / kh);
        float v = 0.f;
        if (c < ic)
            v = src[(((size_t)o * ic + c) * kh + fy) * kw + fx];
        const float h = round_tf32(v);
        dst[i] = h;
        dst[plane + i] = round_tf32(__fsub_rn(v, h));
    }
}

// ------------------------------------------------------------------------------------------
// epilogue
// ------------------------------------------------------------------------------------------
struct F32Epilogue {
    int oc, act;
    const float* bias;
    const float* z;  // optional tensor added after the activation (residual), or nullptr
    long long z_pitch;
    float* dst;
    long long dst_pitch;  // floats between consecutive pixels of dst (>= oc)
};

__device__ __forceinline__ float act_f32(int act, float x) {
    switch (act) {
        case MB200_F32_RELU:
            return x > 0.f ? x : 0.f;
        case MB200_F32_SIGMOID:
            return __fdividef(1.f, 1.f + __expf(-x));
        case MB200_F32_SILU:
            return __fdividef(x, 1.f + __expf(-x));
        case MB200_F32_H_SWISH: {
            float t = x + 3.f;
            t = t > 0.f ? t : 0.f;
            t = t > 6.f ? 6.f : t;
            return x * t * (1.f / 6.f);
        }
        default:
            return x;
    }
}

// 32 consecutive channels (from ch0) of pixel `m`
__device__ __forceinline__ void store_f32_chunk(
        const float (&v)[32], const F32Epilogue& e, size_t m, int ch0) {
    float* out = e.dst + m * e.dst_pitch + ch0;
    const float* zin = e.z ? e.z + m * e.z_pitch + ch0 : nullptr;
    const bool vec = ch0 + 32 <= e.oc && (((uintptr_t)out | (uintptr_t)zin) & 15) == 0 &&
                     (!e.bias || ((uintptr_t)(e.bias + ch0) & 15) == 0);
    if (vec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
            if (e.bias)
                b = __ldg(reinterpret_cast<const float4*>(e.bias + ch0) + j);
            float4 r;
            r.x = act_f32(e.act, v[4 * j + 0] + b.x);
            r.y = act_f32(e.act, v[4 * j + 1] + b.y);
            r.z = act_f32(e.act, v[4 * j + 2] + b.z);
            r.w = act_f32(e.act, v[4 * j + 3] + b.w);
            if (zin) {
                const float4 zz = __ldg(reinterpret_cast<const float4*>(zin) + j);
                r.x += zz.x; r.y += zz.y; r.z += zz.z; r.w += zz.w;
            }
            reinterpret_cast<float4*>(out)[j] = r;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if (ch0 + i < e.oc) {
                float r = act_f32(e.act, v[i] + (e.bias ? e.bias[ch0 + i] : 0.f));
                if (zin)
                    r += zin[i];
                out[i] = r;
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// the tensor-core kernel
// ------------------------------------------------------------------------------------------
struct F32ConvParams {
    int m_total, oc, oh, ow;
    int cblocks;  // row-sized channel blocks per tap
    int taps_w;
    int k_iters;
    int seg_iters;  // pipeline steps per accumulation segment
    int sh, sw, base_h, base_w;
    int m_tiles, n_tiles;
    int a_tiled;      // 1x1, stride 1, no padding: A is the plain matrix [pixels][channels]
    int b_lo_offset;  // rows from the hi plane to the lo plane of the filter
    F32Epilogue ep;
    int* status;
    long long wait_cycles;
};

template <int BN, int ROWB>
struct F32Smem {
    static constexpr int kStages = ROWB == 128 ? (BN == 128 ? 3 : 4) : 6;
    static constexpr int kABytes = kBM * ROWB;
    static constexpr int kBBytes = BN * ROWB;
    static constexpr int kStageBytes = 2 * kABytes + 2 * kBBytes;
    static constexpr int kTiles = kStages * kStageBytes;
    static constexpr int kBarOff = kTiles;
    static constexpr int kTotal = kBarOff + (3 * kMaxStages + 5) * 8 + 16;
    static constexpr int kDynamic = kTotal + 1024;
};

// Eight epilogue warps (two 32-column chunks each for BN = 128). Sixteen, one chunk each,
// halve a warp's chain of dependent TMEM loads per hand-over, but measured no faster on the
// ConvBias layers and 10 % slower on the 4096^3 MatrixMul.
__host__ __device__ constexpr int f32_epilogue_warps(int bn) { return bn >= 64 ? 8 : 8; }
constexpr int kF32ConvertWarps = 4;
__host__ __device__ constexpr int f32_threads(int bn) { return 64 + 32 * f32_epilogue_warps(bn) + 32 * kF32ConvertWarps; }

// v = hi + lo with both halves exact tf32 values (which way a tie rounds does not matter:
// v - hi is exact, and lo is its nearest tf32)
__device__ __forceinline__ void split_tf32(float v, float& hi, float& lo) {
    uint32_t h, l;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(v));
    hi = __uint_as_float(h);
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(__fsub_rn(v, hi)));
    lo = __uint_as_float(l);
}

template <int BN, int ROWB>
__global__ void __launch_bounds__(f32_threads(BN), 1) conv_f32_umma_kernel(
        const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
        const F32ConvParams p) {
    using L = F32Smem<BN, ROWB>;
    constexpr int kSt = L::kStages;
    constexpr int kChans = ROWB / 4;  // floats per row
    constexpr int kF32EpilogueWarps = f32_epilogue_warps(BN);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = (uint64_t*)(smem + L::kBarOff);
    uint64_t* empty_bar = full_bar + kMaxStages;
    uint64_t* conv_bar = empty_bar + kMaxStages;  // the stage's A tile is split: MMAs may read it
    uint64_t* acc_full = conv_bar + kMaxStages;  // [2]
    uint64_t* acc_empty = acc_full + 2;           // [2]
    uint64_t* drain_bar = acc_empty + 2;
    uint32_t* tmem_slot = (uint32_t*)(drain_bar + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_tiles = p.m_tiles * p.n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
            mbar_init(&conv_bar[s], 32 * kF32ConvertWarps);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 32 * kF32EpilogueWarps);
        }
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile(
                "tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                        smem_u32(tmem_slot)),
                "r"(4 * BN)
                : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    pdl_start();  // set-up done: from here on the kernel touches global memory

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int tile_n = tile % p.n_tiles, tile_m = tile / p.n_tiles;
                const int m0 = tile_m * kBM, n0 = tile_n * BN;
                const int img = m0 / (p.oh * p.ow);
                const int rem = m0 - img * (p.oh * p.ow);
                const int oy = rem / p.ow, ox = rem - oy * p.ow;
                const int base_w = ox * p.sw + p.base_w, base_h = oy * p.sh + p.base_h;
                int cb = 0, fx = 0, fy = 0;
                for (int it = 0; it < p.k_iters; ++it) {
                    if (!mbar_wait(&empty_bar[s], phase ^ 1u, abort_flag, p.wait_cycles)) {
                        if (!*abort_flag) {
                            *abort_flag = 1;
                            atomicExch(p.status, ERR_PRODUCER_WAIT);
                        }
                        ok = false;
                        break;
                    }
                    // the fp32 A tile lands in the hi slot; the lo slot is filled on chip
                    mbar_expect_tx(&full_bar[s], (uint32_t)(L::kABytes + 2 * L::kBBytes));
                    uint8_t* a_hi = smem + s * L::kStageBytes;
                    uint8_t* a_lo = a_hi + L::kABytes;
                    uint8_t* b_hi = a_lo + L::kABytes;
                    uint8_t* b_lo = b_hi + L::kBBytes;
                    if (p.a_tiled)
                        tma_load_2d(a_hi, &map_a, &full_bar[s], cb * kChans, m0);
                    else
                        tma_load_im2col_4d(a_hi, &map_a, &full_bar[s], cb * kChans, base_w, base_h,
                                           img, (uint16_t)fx, (uint16_t)fy);
                    tma_load_2d(b_hi, &map_b, &full_bar[s], it * kChans, n0);
                    tma_load_2d(b_lo, &map_b, &full_bar[s], it * kChans, n0 + p.b_lo_offset);
                    if (++cb == p.cblocks) {
                        cb = 0;
                        if (++fx == p.taps_w) {
                            fx = 0;
                            ++fy;
                        }
                    }
                    if (++s == kSt) {
                        s = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_tf32(kBM, BN);
            // swizzled K-major tiles: 8-row groups 8 * ROWB bytes apart
            constexpr uint32_t kLayout = ROWB == 128 ? 2u : 4u;
            constexpr uint32_t kSbo = 8 * ROWB;
            int local = 0, s = 0;  // `local` counts accumulation segments
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                for (int k0 = 0; k0 < p.k_iters && ok; k0 += p.seg_iters, ++local) {
                    const int k1 = min(k0 + p.seg_iters, p.k_iters);
                    const int buf = local & 1;
                    const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
                    if (!mbar_wait(&acc_empty[buf], acc_phase ^ 1u, abort_flag, p.wait_cycles)) {
                        if (!*abort_flag) {
                            *abort_flag = 1;
                            atomicExch(p.status, ERR_MMA_ACC_WAIT);
                        }
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    // main sum (hi * hi) and correction sum (lo * hi + hi * lo) of this set
                    const uint32_t tmem_d = tmem_base + (uint32_t)(buf * 2 * BN);
                    const uint32_t tmem_c = tmem_d + (uint32_t)BN;
                    for (int it = k0; it < k1; ++it) {
                        if (!mbar_wait(&conv_bar[s], phase, abort_flag, p.wait_cycles)) {
                            if (!*abort_flag) {
                                *abort_flag = 1;
                                atomicExch(p.status, ERR_MMA_WAIT);
                            }
                            ok = false;
                            break;
                        }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t a_addr = smem_u32(smem + s * L::kStageBytes);
                        const uint64_t a_hi = umma_smem_desc(a_addr, 16, kSbo, kLayout);
                        const uint64_t a_lo =
                                umma_smem_desc(a_addr + L::kABytes, 16, kSbo, kLayout);
                        const uint64_t b_hi =
                                umma_smem_desc(a_addr + 2 * L::kABytes, 16, kSbo, kLayout);
                        const uint64_t b_lo = umma_smem_desc(
                                a_addr + 2 * L::kABytes + L::kBBytes, 16, kSbo, kLayout);
                        // a K step of 8 floats is 32 bytes inside the swizzled row: +2 in the
                        // descriptor's 16-byte address units
                        const uint32_t acc = it != k0 ? 1u : 0u;
                        umma_tf32(tmem_c, a_lo, b_hi, idesc, acc);
                        umma_tf32_c<true>(tmem_c, a_hi, b_lo, idesc);
                        umma_tf32(tmem_d, a_hi, b_hi, idesc, acc);
#pragma unroll
                        for (int k = 1; k < ROWB / 32; ++k) {
                            umma_tf32_c<true>(tmem_c, a_lo + 2 * k, b_hi + 2 * k, idesc);
                            umma_tf32_c<true>(tmem_c, a_hi + 2 * k, b_lo + 2 * k, idesc);
                            umma_tf32_c<true>(tmem_d, a_hi + 2 * k, b_hi + 2 * k, idesc);
                        }
                        umma_commit(&empty_bar[s]);
                        if (++s == kSt) {
                            s = 0;
                            phase ^= 1u;
                        }
                    }
                    if (ok)
                        umma_commit(&acc_full[buf]);
                }
            }
        }
    } else if (warp >= 2 + kF32EpilogueWarps) {
        // ---------------- converters: fp32 A tile -> hi (in place) and lo planes ----------------
        const int ct = (int)threadIdx.x - (64 + 32 * kF32EpilogueWarps);
        constexpr int kVecs = L::kABytes / 16;
        constexpr int kPerThread = kVecs / (32 * kF32ConvertWarps);
        static_assert(kVecs % (32 * kF32ConvertWarps) == 0, "whole vectors per converter thread");
        int s = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            for (int it = 0; it < p.k_iters; ++it) {
                ok = mbar_wait(&full_bar[s], phase, abort_flag, p.wait_cycles);
                if (!ok && !*abort_flag) {
                    *abort_flag = 1;
                    atomicExch(p.status, ERR_PRODUCER_WAIT);
                }
                ok = __all_sync(0xffffffffu, ok);
                if (!ok)
                    break;
                float4* hi = reinterpret_cast<float4*>(smem + s * L::kStageBytes);
                float4* lo = hi + kVecs;
#pragma unroll
                for (int j = 0; j < kPerThread; ++j) {
                    const int idx = ct + j * 32 * kF32ConvertWarps;
                    const float4 v = hi[idx];
                    float4 h, l;
                    split_tf32(v.x, h.x, l.x);
                    split_tf32(v.y, h.y, l.y);
                    split_tf32(v.z, h.z, l.z);
                    split_tf32(v.w, h.w, l.w);
                    hi[idx] = h;
                    lo[idx] = l;
                }
                // generic-proxy writes, read next by the tensor core through the async proxy
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(&conv_bar[s]);
                if (++s == kSt) {
                    s = 0;
                    phase ^= 1u;
                }
            }
        }
    } else {
        // ---------------- epilogue: warps 2..9, TMEM lanes 32 * (warp % 4) .. ----------------
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const int half = (warp - 2) >> 2;
        constexpr int kChunksPerWarp = (BN / 32) / (kF32EpilogueWarps / 4);
        static_assert(kChunksPerWarp >= 1, "every epilogue warp must own a chunk");
        int local = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const int tile_n = tile % p.n_tiles, tile_m = tile / p.n_tiles;
            const int m = tile_m * kBM + row, n0 = tile_n * BN;
            // running fp32 sums of this thread's accumulators over the tile's segments
            float sum[kChunksPerWarp][32];
            for (int k0 = 0; k0 < p.k_iters && ok; k0 += p.seg_iters, ++local) {
                const int buf = local & 1;
                const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
                ok = mbar_wait(&acc_full[buf], acc_phase, abort_flag, p.wait_cycles);
                if (!ok && !*abort_flag) {
                    *abort_flag = 1;
                    atomicExch(p.status, ERR_EPILOGUE_WAIT);
                }
                ok = __all_sync(0xffffffffu, ok);
                if (!ok)
                    break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t taddr =
                        tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * 2 * BN);
#pragma unroll
                for (int cc = 0; cc < kChunksPerWarp; ++cc) {
                    const uint32_t col = (uint32_t)((half * kChunksPerWarp + cc) * 32);
                    uint32_t v[32];
                    tmem_ld32(taddr + col, v);  // main sum
                    if (k0 == 0) {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            sum[cc][j] = __uint_as_float(v[j]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            sum[cc][j] = __fadd_rn(sum[cc][j], __uint_as_float(v[j]));
                    }
                    tmem_ld32(taddr + (uint32_t)BN + col, v);  // correction sum
                    if (cc + 1 == kChunksPerWarp) {
                        // this thread's accumulators are in registers: hand the set back
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        mbar_arrive(&acc_empty[buf]);
                    }
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        sum[cc][j] = __fadd_rn(sum[cc][j], __uint_as_float(v[j]));
                }
            }
            if (!ok)
                break;
#pragma unroll
            for (int cc = 0; cc < kChunksPerWarp; ++cc) {
                const int ch0 = n0 + (half * kChunksPerWarp + cc) * 32;
                if (m < p.m_total && ch0 < p.oc)
                    store_f32_chunk(sum[cc], p.ep, (size_t)m, ch0);
            }
        }
    }

    // ---------------- teardown ----------------
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_flag) {
        if (warp == 1 && lane == 0) {
            umma_commit(drain_bar);
            const long long t0 = clock64();
            while (!mbar_try_wait(drain_bar, 0)) {
                if (clock64() - t0 > p.wait_cycles) {
                    atomicExch(p.status, ERR_DRAIN_WAIT);
                    break;
                }
            }
        }
        for (int i = 0; i < 200; ++i)
            __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(4 * BN)
                     : "memory");
    }
}

// ------------------------------------------------------------------------------------------
// general CUDA-core kernel: any shape, groups, odd channel counts; also the small heads
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) conv_f32_direct_kernel(
        ConvF32Args a, const float* __restrict__ src, const float* __restrict__ flt,
        const float* __restrict__ bias, const float* __restrict__ z, float* __restrict__ dst) {
    pdl_start();
    // flt: the unsplit K-major filter [OC][KH][KW][ICpg]
    const size_t total = (size_t)a.m * a.oc;
    const int icpg = a.ic / a.groups, ocpg = a.oc / a.groups;
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int o = (int)(idx % a.oc);
        const size_t m = idx / a.oc;
        const int ox = (int)(m % a.ow);
        const size_t t = m / a.ow;
        const int oy = (int)(t % a.oh);
        const int n = (int)(t / a.oh);
        const int g = o / ocpg;
        const float* w = flt + (size_t)o * a.kh * a.kw * icpg;
        float acc = 0.f;
        for (int fy = 0; fy < a.kh; ++fy) {
            const int iy = oy * a.sh + fy - a.ph;
            if ((unsigned)iy >= (unsigned)a.ih)
                continue;
            for (int fx = 0; fx < a.kw; ++fx) {
                const int ix = ox * a.sw + fx - a.pw;
                if ((unsigned)ix >= (unsigned)a.iw)
                    continue;
                const float* s = src + (((size_t)n * a.ih + iy) * a.iw + ix) * a.src_pitch +
                                 g * icpg;
                const float* wk = w + (size_t)(fy * a.kw + fx) * icpg;
                for (int c = 0; c < icpg; ++c)
                    acc = fmaf(s[c], wk[c], acc);
            }
        }
        float r = act_f32(a.act, acc + (bias ? bias[o] : 0.f));
        if (z)
            r += z[m * a.z_pitch + o];
        dst[m * a.dst_pitch + o] = r;
    }
}

// OIHW / [G][OCpg][ICpg][KH][KW] fp32 -> [OC][KH][KW][ICpg]
__global__ void __launch_bounds__(256) pack_filter_f32_plain_kernel(
        const float* __restrict__ src, float* __restrict__ dst, int oc, int icpg, int kh, int kw) {
    const size_t total = (size_t)oc * icpg * kh * kw;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % icpg);
        size_t t = i / icpg;
        const int fx = (int)(t % kw);
        t /= kw;
        const int fy = (int)(t % kh);
        const int o = (int)(t / kh);
        dst[i] = src[(((size_t)o * icpg + c) * kh + fy) * kw + fx];
    }
}

int grid_1d(size_t work, int block) {
    size_t g = (work + block - 1) / block;
    const size_t most = (size_t)sm_count() * 16;
    if (g > most)
        g = most;
    return g < 1 ? 1 : (int)g;
}

template <int BN, int ROWB>
int launch_f32_kernel(
        const CUtensorMap& ma, const CUtensorMap& mb, const F32ConvParams& p, cudaStream_t st) {
    using L = F32Smem<BN, ROWB>;
    if (cudaFuncSetAttribute(conv_f32_umma_kernel<BN, ROWB>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             L::kDynamic) != cudaSuccess)
        return check_launch("conv_f32_umma smem attribute");
    constexpr int kF32Threads = f32_threads(BN);
    const int per_sm = resident_ctas_per_sm(conv_f32_umma_kernel<BN, ROWB>, kF32Threads,
                                            L::kDynamic, 4 * BN);
    const int total = p.m_tiles * p.n_tiles;
    int grid = sm_count() * per_sm;
    if (grid > total)
        grid = total;
    if (tuning().debug)
        fprintf(stderr, "conv_f32_umma<%d,%d>: per_sm %d grid %d tiles %d k_iters %d smem %d\n", BN,
                ROWB, per_sm, grid, total, p.k_iters, L::kDynamic);
    launch_pdl(conv_f32_umma_kernel<BN, ROWB>, dim3(grid), dim3(kF32Threads), (size_t)L::kDynamic, st,
               ma, mb, p);
    return check_launch("conv_f32_umma");
}

bool plain_matrix(const ConvF32Args& a) {
    return a.kh == 1 && a.kw == 1 && a.sh == 1 && a.sw == 1 && a.ph == 0 && a.pw == 0;
}

}  // namespace

// channels the packed (split) filter holds per tap: ic rounded up to a whole TMA row
int conv_f32_padded_ic(int ic) {
    return ic <= 16 ? 16 : (ic + 31) / 32 * 32;
}

size_t conv_f32_split_filter_floats(const ConvF32Args& a) {
    return 2 * (size_t)a.oc * a.kh * a.kw * conv_f32_padded_ic(a.ic);
}

// Tensor-core path: dense, channel count a whole number of TMA rows (16, or a multiple of 32
// floats), the source a contiguous NHWC tensor of at least 128 KiB, 16-byte aligned operands.
bool conv_f32_umma_supported(const ConvF32Args& a, const float* src, const float* dst) {
    if (a.groups != 1)
        return false;
    if (!(a.ic == 16 || a.ic % 32 == 0))
        return false;
    if (a.src_pitch != a.ic)
        return false;
    if (a.kh * a.kw > 49 || a.ph > 64 || a.pw > 64 || a.sh > 8 || a.sw > 8)
        return false;
    if ((size_t)a.n * a.ih * a.iw * a.ic * 4 < 131072)
        return false;
    if ((size_t)a.n * a.ih * a.iw >= (1ull << 31) || (size_t)a.m >= (1ull << 31))
        return false;
    if (((uintptr_t)src | (uintptr_t)dst) & 15)
        return false;
    if ((a.dst_pitch & 3) || (a.z_pitch & 3))
        return false;
    return true;
}

size_t conv_f32_workspace_bytes(const ConvF32Args& a) {
    (void)a;  // the activation is split into its tf32 planes in shared memory
    return 0;
}

int launch_conv_f32_pack_filter_split(
        const ConvF32Args& a, const float* flt_oihw, float* out, cudaStream_t st) {
    const int icp = conv_f32_padded_ic(a.ic);
    const size_t plane = (size_t)a.oc * a.kh * a.kw * icp;
    pack_filter_f32_kernel<<<grid_1d(plane, 256), 256, 0, st>>>(flt_oihw, out, a.oc, a.ic, icp,
                                                                 a.kh, a.kw);
    return check_launch("pack_filter_f32");
}

int launch_conv_f32_pack_filter_plain(
        const ConvF32Args& a, const float* flt_oihw, float* out, cudaStream_t st) {
    const int icpg = a.ic / a.groups;
    const size_t total = (size_t)a.oc * icpg * a.kh * a.kw;
    pack_filter_f32_plain_kernel<<<grid_1d(total, 256), 256, 0, st>>>(flt_oihw, out, a.oc, icpg,
                                                                       a.kh, a.kw);
    return check_launch("pack_filter_f32_plain");
}

int launch_conv_f32_direct(
        const ConvF32Args& a, const float* src, const float* flt_plain, const float* bias,
        const float* z, float* dst, cudaStream_t st) {
    launch_pdl(conv_f32_direct_kernel, dim3(grid_1d((size_t)a.m * a.oc, 256)), dim3(256), 0, st, a,
               src, flt_plain, bias, z, dst);
    return check_launch("conv_f32_direct");
}

int launch_conv_f32_umma(
        const ConvF32Args& a, const float* src, const float* flt_split, const float* bias,
        const float* z, float* dst, void* workspace, cudaStream_t st) {
    const DriverApi& api = driver_api();
    if (!api.ok)
        return set_error(ST_RUNTIME, "cuTensorMapEncode* entry points not found in the driver");
    (void)workspace;  // the operands are split in shared memory: no scratch tensor
    if ((uintptr_t)flt_split & 15)
        return set_error(ST_INVALID_LAYOUT, "the filter must be 16-byte aligned");

    const int rowb = a.ic == 16 ? 64 : 128;
    const int chans = rowb / 4;
    const CUtensorMapSwizzle swz =
            rowb == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
    const int bn = a.oc <= 64 ? 64 : 128;
    const int taps = a.kh * a.kw;
    const bool a_tiled = plain_matrix(a);
    CUtensorMap map_a, map_b;
    if (a_tiled) {
        cuuint64_t dims[2] = {(cuuint64_t)a.ic, (cuuint64_t)a.m};
        cuuint64_t strides[1] = {(cuuint64_t)a.ic * 4};
        cuuint32_t box[2] = {(cuuint32_t)chans, (cuuint32_t)kBM};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = api.tiled(&map_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)src, dims, strides,
                               box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return set_error(ST_RUNTIME, "cuTensorMapEncodeTiled(f32 activation) failed: %d", (int)r);
    } else {
        cuuint64_t dims[4] = {(cuuint64_t)a.ic, (cuuint64_t)a.iw, (cuuint64_t)a.ih,
                              (cuuint64_t)a.n};
        cuuint64_t strides[3] = {(cuuint64_t)a.ic * 4, (cuuint64_t)a.iw * a.ic * 4,
                                 (cuuint64_t)a.ih * a.iw * a.ic * 4};
        int lower[2] = {-a.pw, -a.ph};
        int upper[2] = {(a.ow - 1) * a.sw - a.pw - (a.iw - 1), (a.oh - 1) * a.sh - a.ph - (a.ih - 1)};
        cuuint32_t estr[4] = {1, (cuuint32_t)a.sw, (cuuint32_t)a.sh, 1};
        CUresult r = api.im2col(&map_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void*)src, dims, strides,
                                lower, upper, chans, kBM, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return set_error(ST_RUNTIME, "cuTensorMapEncodeIm2col(f32) failed: %d", (int)r);
    }
    {
        const cuuint64_t k_total = (cuuint64_t)taps * a.ic;
        cuuint64_t dims[2] = {k_total, (cuuint64_t)2 * a.oc};
        cuuint64_t strides[1] = {k_total * 4};
        cuuint32_t box[2] = {(cuuint32_t)chans, (cuuint32_t)bn};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = api.tiled(&map_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)flt_split, dims,
                               strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return set_error(ST_RUNTIME, "cuTensorMapEncodeTiled(f32 filter) failed: %d", (int)r);
    }
    F32ConvParams p;
    p.m_total = a.m;
    p.oc = a.oc;
    p.oh = a.oh;
    p.ow = a.ow;
    p.cblocks = a.ic / chans;
    p.taps_w = a.kw;
    p.k_iters = taps * p.cblocks;
    // eight K = 8 steps per TMEM accumulation chain
    p.seg_iters = 8 / (rowb / 32);
    p.sh = a.sh;
    p.sw = a.sw;
    p.base_h = -a.ph;
    p.base_w = -a.pw;
    p.m_tiles = (a.m + kBM - 1) / kBM;
    p.n_tiles = (a.oc + bn - 1) / bn;
    p.a_tiled = a_tiled ? 1 : 0;
    p.b_lo_offset = a.oc;
    p.ep.oc = a.oc;
    p.ep.act = a.act;
    p.ep.bias = bias;
    p.ep.z = z;
    p.ep.z_pitch = a.z_pitch;
    p.ep.dst = dst;
    p.ep.dst_pitch = a.dst_pitch;
    p.status = device_status_word(st);
    if (!p.status)
        return ST_MALLOC;
    p.wait_cycles = kWaitCycles;
    if (rowb == 128)
        return bn == 64 ? launch_f32_kernel<64, 128>(map_a, map_b, p, st)
                        : launch_f32_kernel<128, 128>(map_a, map_b, p, st);
    return bn == 64 ? launch_f32_kernel<64, 64>(map_a, map_b, p, st)
                    : launch_f32_kernel<128, 64>(map_a, map_b, p, st);
}

}  // namespace mb200
