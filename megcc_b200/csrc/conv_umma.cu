// qint8 ConvBias as implicit GEMM on the sm_100a tensor cores.
//
//   D[m, oc] = sum_{fy,fx,c} A[m, (fy,fx,c)] * W[oc, (fy,fx,c)],   m = (n, oh, ow) linearised
//
// * activations NHWC int8; one TMA im2col load per (filter tap, 64-channel block) brings the
//   128 consecutive output pixels of the tile straight into a 64B-swizzled K-major tile
//   (padding and stride are resolved by the im2col bounding box / traversal stride);
// * filter pre-packed [OC][KH][KW][IC], fetched by a tiled 2D TMA into the same swizzle;
// * tcgen05.mma kind::i8, M=128 x N=BN x K=32 per instruction, int32 accumulators in TMEM;
// * warp roles: warp 0 = TMA producer, warp 1 = MMA issuer (+ TMEM alloc), warps 2..5 =
//   epilogue (tcgen05.ld -> +bias -> fp32 requant in the reference's operation order ->
//   activation -> int8 -> 16-byte stores);
// * every wait is bounded: when it runs out the kernel records a code in the device status
//   word, drains what it started, frees its TMEM and returns.
//
// Replaces the loop nest of compiler/lib/KernelGen/BareMetal/ConvKernel.cpp:305-344 and
// its epilogue (:374-382, BareMetal/Activation.cpp:105-113) for dense convolutions whose
// input channel count is a multiple of 64.
#include <cuda.h>

#include "internal.h"

namespace mb200 {

namespace {

constexpr int kBM = 128;         // output pixels per tile (UMMA M)
constexpr int kBK = 64;          // K bytes per pipeline stage = channels per TMA row
constexpr int kUmmaK = 32;       // K per tcgen05.mma kind::i8
constexpr int kStages = 6;
constexpr int kThreads = 192;
constexpr long long kWaitCycles = 1LL << 31;  // ~1 s: only a lost barrier gets there

enum : int {
    ERR_PRODUCER_WAIT = 0x101,
    ERR_MMA_WAIT = 0x102,
    ERR_EPILOGUE_WAIT = 0x103,
    ERR_DRAIN_WAIT = 0x104,
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
    return ok != 0;
}

// Bounded wait. Returns false when the limit ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(
        uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity))
        return true;
    const long long t0 = clock64();
    for (int spin = 0;; ++spin) {
        if (mbar_try_wait(bar, parity))
            return true;
        if ((spin & 255) == 255) {
            if (*abort_flag)
                return false;
            if (clock64() - t0 > kWaitCycles)
                return false;
        }
    }
}

__device__ __forceinline__ void tma_load_2d(
        void* smem, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem)),
            "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
            : "memory");
}

__device__ __forceinline__ void tma_load_im2col_4d(
        void* smem, const CUtensorMap* map, uint64_t* bar, int c, int w, int h, int n,
        uint16_t off_w, uint16_t off_h) {
    asm volatile(
            "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};" ::"r"(smem_u32(smem)),
            "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w),
            "h"(off_h)
            : "memory");
}

// K-major operand tile with 64-byte swizzle: rows of 64 bytes, 8-row groups 512 bytes apart.
__device__ __forceinline__ uint64_t umma_smem_desc_sw64(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);  // start address, 16-byte units
    d |= (uint64_t)1 << 16;                    // leading byte offset: unused with swizzle
    d |= (uint64_t)(512 >> 4) << 32;           // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                    // descriptor version of sm_100
    d |= (uint64_t)4 << 61;                    // layout type SWIZZLE_64B
    return d;
}

// kind::i8 instruction descriptor: int32 accumulate, signed 8-bit A and B, both K-major.
__host__ __device__ constexpr uint32_t umma_idesc_s8(int m, int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_s8(
        uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile(
            "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                    smem_u32(bar))
            : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, "
            "[%32];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
              "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]),
              "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
              "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
              "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
              "=r"(v[31])
            : "r"(taddr)
            : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

struct UmmaConvParams {
    int m_total, oc, oh, ow, ic;
    int kh, kw, sh, sw, ph, pw, dh, dw;
    int n_tiles;
    int act;
    float s_src, s_flt, s_dst;
    const int32_t* bias;
    const float* flt_scales;
    int8_t* dst;
    int* status;
};

template <int BN>
struct SmemLayout {
    static constexpr int kABytes = kBM * kBK;
    static constexpr int kBBytes = BN * kBK;
    static constexpr int kTiles = kStages * (kABytes + kBBytes);
    // after the tiles: full[kStages], empty[kStages], accum, drain barriers, bias, scales
    static constexpr int kBarOff = kTiles;
    static constexpr int kBiasOff = kBarOff + (2 * kStages + 2) * 8 + 16;
    static constexpr int kScaleOff = kBiasOff + BN * 4;
    static constexpr int kTotal = kScaleOff + BN * 4;
    static constexpr int kDynamic = kTotal + 1024;  // room to align the tiles to 1024 bytes
};

template <int BN>
__global__ void __launch_bounds__(kThreads) conv_umma_kernel(
        const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
        const UmmaConvParams p) {
    using L = SmemLayout<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* tiles_a = smem;
    uint8_t* tiles_b = smem + kStages * L::kABytes;
    uint64_t* full_bar = (uint64_t*)(smem + L::kBarOff);
    uint64_t* empty_bar = full_bar + kStages;
    uint64_t* accum_bar = empty_bar + kStages;
    uint64_t* drain_bar = accum_bar + 1;
    uint32_t* tmem_slot = (uint32_t*)(drain_bar + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    int32_t* s_bias = (int32_t*)(smem + L::kBiasOff);
    float* s_scale = (float*)(smem + L::kScaleOff);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_n = blockIdx.x % p.n_tiles, tile_m = blockIdx.x / p.n_tiles;
    const int m0 = tile_m * kBM, n0 = tile_n * BN;
    const int cblocks = p.ic / kBK;
    const int k_iters = p.kh * p.kw * cblocks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(accum_bar, 1);
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile(
                "tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                        smem_u32(tmem_slot)),
                "r"(BN)
                : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // bias / per-channel scales of this tile's channels
    for (int i = threadIdx.x; i < BN; i += kThreads) {
        const int ch = n0 + i;
        s_bias[i] = (p.bias && ch < p.oc) ? p.bias[ch] : 0;
        s_scale[i] = (p.flt_scales && ch < p.oc) ? p.flt_scales[ch] : p.s_flt;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            const int img = m0 / (p.oh * p.ow);
            const int rem = m0 - img * (p.oh * p.ow);
            const int oy = rem / p.ow, ox = rem - oy * p.ow;
            const int base_w = ox * p.sw - p.pw, base_h = oy * p.sh - p.ph;
            for (int it = 0; it < k_iters; ++it) {
                const int s = it % kStages;
                const uint32_t phase = (uint32_t)(it / kStages) & 1u;
                if (!mbar_wait(&empty_bar[s], phase ^ 1u, abort_flag)) {
                    if (!*abort_flag) {
                        *abort_flag = 1;
                        atomicExch(p.status, ERR_PRODUCER_WAIT);
                    }
                    break;
                }
                const int tap = it / cblocks, cb = it - tap * cblocks;
                const int fy = tap / p.kw, fx = tap - fy * p.kw;
                mbar_expect_tx(&full_bar[s], (uint32_t)(L::kABytes + L::kBBytes));
                tma_load_im2col_4d(
                        tiles_a + s * L::kABytes, &map_a, &full_bar[s], cb * kBK, base_w, base_h,
                        img, (uint16_t)(fx * p.dw), (uint16_t)(fy * p.dh));
                tma_load_2d(tiles_b + s * L::kBBytes, &map_b, &full_bar[s], it * kBK, n0);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_s8(kBM, BN);
            bool ok = true;
            for (int it = 0; it < k_iters && ok; ++it) {
                const int s = it % kStages;
                const uint32_t phase = (uint32_t)(it / kStages) & 1u;
                if (!mbar_wait(&full_bar[s], phase, abort_flag)) {
                    if (!*abort_flag) {
                        *abort_flag = 1;
                        atomicExch(p.status, ERR_MMA_WAIT);
                    }
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t adesc = umma_smem_desc_sw64(smem_u32(tiles_a + s * L::kABytes));
                const uint64_t bdesc = umma_smem_desc_sw64(smem_u32(tiles_b + s * L::kBBytes));
#pragma unroll
                for (int k = 0; k < kBK / kUmmaK; ++k) {
                    // +32 bytes along K inside the swizzle row = +2 in the address field
                    umma_s8(tmem_base, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2),
                            idesc, (it | k) != 0 ? 1u : 0u);
                }
                umma_commit(&empty_bar[s]);  // frees the stage once these MMAs retire
            }
            if (ok)
                umma_commit(accum_bar);
        }
    } else {
        // ---------------- epilogue: warps 2..5 own TMEM lanes 32*(warp%4).. ----------------
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const int m = m0 + row;
        bool ok = mbar_wait(accum_bar, 0, abort_flag);
        if (!ok && !*abort_flag) {
            *abort_flag = 1;
            atomicExch(p.status, ERR_EPILOGUE_WAIT);
        }
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const bool vec_ok = (p.oc % 16) == 0;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32), v);
                const int ch0 = n0 + c * 32;
                if (m < p.m_total && ch0 < p.oc) {
                    uint32_t packed[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        int r[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int i = c * 32 + j * 4 + e;
                            const int acc = (int)v[j * 4 + e] + s_bias[i];
                            r[e] = requant_conv(acc, p.s_src, s_scale[i], p.s_dst, p.act);
                        }
                        packed[j] = pack4(r[0], r[1], r[2], r[3]);
                    }
                    int8_t* out = p.dst + (size_t)m * p.oc + ch0;
                    if (vec_ok && ch0 + 32 <= p.oc) {
                        reinterpret_cast<uint4*>(out)[0] =
                                make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        reinterpret_cast<uint4*>(out)[1] =
                                make_uint4(packed[4], packed[5], packed[6], packed[7]);
                    } else {
                        for (int i = 0; i < 32 && ch0 + i < p.oc; ++i)
                            out[i] = (int8_t)(packed[i >> 2] >> (8 * (i & 3)));
                    }
                }
            }
        }
    }

    // ---------------- teardown ----------------
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_flag) {
        // a wait ran out: let loads in flight land and MMAs retire (both bounded) before
        // the shared memory and TMEM are given back
        if (warp == 1 && lane == 0) {
            umma_commit(drain_bar);
            const long long t0 = clock64();
            while (!mbar_try_wait(drain_bar, 0)) {
                if (clock64() - t0 > kWaitCycles) {
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
                     "r"(BN)
                     : "memory");
    }
}

// ------------------------------------------------------------------------------------------
// host side: tensor maps and launch
// ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(
        CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
        const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
        CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(
        CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
        const cuuint64_t*, const int*, const int*, cuuint32_t, cuuint32_t, const cuuint32_t*,
        CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
        CUtensorMapFloatOOBfill);

struct DriverApi {
    EncodeTiledFn tiled = nullptr;
    EncodeIm2colFn im2col = nullptr;
    bool ok = false;
};

const DriverApi& driver_api() {
    static DriverApi api = [] {
        DriverApi a;
        cudaDriverEntryPointQueryResult q;
        void* f = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) ==
                    cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            a.tiled = (EncodeTiledFn)f;
        f = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &f, cudaEnableDefault, &q) ==
                    cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            a.im2col = (EncodeIm2colFn)f;
        a.ok = a.tiled && a.im2col;
        return a;
    }();
    return api;
}

int pick_bn(int oc) {
    return oc <= 64 ? 64 : 128;
}

template <int BN>
int launch_bn(
        const CUtensorMap& ma, const CUtensorMap& mb, const UmmaConvParams& p, int grid,
        cudaStream_t st) {
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(
                    conv_umma_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                    SmemLayout<BN>::kDynamic) != cudaSuccess)
            return check_launch("conv_umma smem attribute");
        attr_set = true;
    }
    conv_umma_kernel<BN><<<grid, kThreads, SmemLayout<BN>::kDynamic, st>>>(ma, mb, p);
    return check_launch("conv_umma");
}

}  // namespace

bool conv_umma_supported(
        const ConvArgs& a, const int8_t* src, const int8_t* flt, const int8_t* dst) {
    if (a.groups != 1 || a.src_is_nchw)
        return false;
    if (a.ic % kBK != 0 || a.oc % 8 != 0)
        return false;
    if (a.kh * a.kw > 49 || a.dh != 1 || a.dw != 1)
        return false;
    // im2col bounding-box corners and tap offsets are 8-bit fields for a 4-D map
    if (a.ph > 64 || a.pw > 64 || a.kh > 64 || a.kw > 64 || a.sh > 8 || a.sw > 8)
        return false;
    // the driver mis-encodes im2col maps of very small tensors; keep those on the
    // general kernel
    if ((size_t)a.n * a.ih * a.iw * a.ic < 131072)
        return false;
    if (((uintptr_t)src | (uintptr_t)flt | (uintptr_t)dst) & 15)
        return false;
    return true;
}

int launch_conv_umma(
        const ConvArgs& a, const int8_t* src, const int8_t* flt, const int32_t* bias,
        const float* flt_scales, int8_t* dst, cudaStream_t st) {
    const DriverApi& api = driver_api();
    if (!api.ok)
        return set_error(ST_RUNTIME, "cuTensorMapEncode* entry points not found in the driver");
    const int bn = pick_bn(a.oc);

    CUtensorMap map_a, map_b;
    {
        cuuint64_t dims[4] = {(cuuint64_t)a.ic, (cuuint64_t)a.iw, (cuuint64_t)a.ih,
                              (cuuint64_t)a.n};
        cuuint64_t strides[3] = {(cuuint64_t)a.ic, (cuuint64_t)a.iw * a.ic,
                                 (cuuint64_t)a.ih * a.iw * a.ic};
        int lower[2] = {-a.pw, -a.ph};
        int upper[2] = {a.pw - (a.kw - 1) * a.dw, a.ph - (a.kh - 1) * a.dh};
        cuuint32_t estr[4] = {1, (cuuint32_t)a.sw, (cuuint32_t)a.sh, 1};
        CUresult r = api.im2col(
                &map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)src, dims, strides, lower, upper,
                kBK, kBM, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return set_error(ST_RUNTIME, "cuTensorMapEncodeIm2col failed: %d", (int)r);
    }
    {
        const cuuint64_t k_total = (cuuint64_t)a.kh * a.kw * a.ic;
        cuuint64_t dims[2] = {k_total, (cuuint64_t)a.oc};
        cuuint64_t strides[1] = {k_total};
        cuuint32_t box[2] = {kBK, (cuuint32_t)bn};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = api.tiled(
                &map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)flt, dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return set_error(ST_RUNTIME, "cuTensorMapEncodeTiled failed: %d", (int)r);
    }

    UmmaConvParams p;
    p.m_total = a.m;
    p.oc = a.oc;
    p.oh = a.oh;
    p.ow = a.ow;
    p.ic = a.ic;
    p.kh = a.kh;
    p.kw = a.kw;
    p.sh = a.sh;
    p.sw = a.sw;
    p.ph = a.ph;
    p.pw = a.pw;
    p.dh = a.dh;
    p.dw = a.dw;
    p.n_tiles = (a.oc + bn - 1) / bn;
    p.act = a.act;
    p.s_src = a.s_src;
    p.s_flt = a.s_flt;
    p.s_dst = a.s_dst;
    p.bias = bias;
    p.flt_scales = flt_scales;
    p.dst = dst;
    p.status = device_status_word();
    if (!p.status)
        return ST_MALLOC;
    const int m_tiles = (a.m + kBM - 1) / kBM;
    const int grid = m_tiles * p.n_tiles;
    return bn == 64 ? launch_bn<64>(map_a, map_b, p, grid, st)
                    : launch_bn<128>(map_a, map_b, p, grid, st);
}

}  // namespace mb200
