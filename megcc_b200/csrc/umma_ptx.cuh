// Inline-PTX building blocks shared by the tensor-core ConvBias kernels: mbarrier waits with
// a time limit, TMA loads (tiled and im2col; no cluster multicast is used anywhere), UMMA
// shared-memory / instruction descriptors, tcgen05.mma / commit / ld.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#ifndef MB200_TRY_WAIT_HINT_NS
#define MB200_TRY_WAIT_HINT_NS 2000
#endif
#ifndef MB200_WAIT_SLEEP_CAP
#define MB200_WAIT_SLEEP_CAP 160
#endif
namespace mb200 {
namespace umma {

constexpr long long kWaitCycles = 1LL << 31;  // ~1 s: only a lost barrier gets there

enum : int {
    ERR_PRODUCER_WAIT = 0x101,
    ERR_MMA_WAIT = 0x102,
    ERR_EPILOGUE_WAIT = 0x103,
    ERR_DRAIN_WAIT = 0x104,
    ERR_MMA_ACC_WAIT = 0x105,
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

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
            "{\n\t.reg .pred p;\n\t"
            // the hint lets the hardware park the thread until the phase completes (or the
            // time passes) instead of burning issue slots in a software spin
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity), "r"((uint32_t)MB200_TRY_WAIT_HINT_NS)
            : "memory");
    return ok != 0;
}

// Bounded wait. Returns false when the limit ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(
        uint64_t* bar, uint32_t parity, volatile int* abort_flag,
        long long limit = kWaitCycles) {
    // A few immediate polls, then short sleeps (20 ns doubling to 160 ns): roles that wait
    // for most of a kernel (producer and MMA thread of an epilogue-bound layer) should not
    // take issue slots from the warps that work. Measured against polling without sleeps on
    // one GPU, neither way changed any kernel's time by more than 1 %.
#pragma unroll 1
    for (int i = 0; i < 8; ++i)
        if (mbar_try_wait(bar, parity))
            return true;
    const long long t0 = clock64();
    unsigned ns = 20;
    for (int spin = 0;; ++spin) {
        if (mbar_try_wait(bar, parity))
            return true;
        __nanosleep(ns);
        if (ns < MB200_WAIT_SLEEP_CAP)
            ns *= 2;
        if ((spin & 63) == 63) {
            if (*abort_flag)
                return false;
            if (clock64() - t0 > limit)
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

__device__ __forceinline__ void tma_load_3d(
        void* smem, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
    asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(smem)),
            "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
            : "memory");
}

__device__ __forceinline__ void tma_load_4d(
        void* smem, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3) {
    asm volatile(
            "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(smem_u32(smem)),
            "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
            : "memory");
}

__device__ __forceinline__ void tma_load_5d(
        void* smem, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3, int c4) {
    asm volatile(
            "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(smem_u32(smem)),
            "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
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

// Shared-memory matrix descriptor of a K-major operand tile.
//   swizzled (64 B): rows of 64 bytes, 8-row groups `sbo` bytes apart, `lbo` unused
//   plain:           8x16-byte core matrices; `lbo` = distance between the two 16-byte K
//                    halves of one MMA, `sbo` = distance between 8-row groups
__device__ __forceinline__ uint64_t umma_smem_desc(
        uint32_t saddr, uint32_t lbo, uint32_t sbo, uint32_t layout_type) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version of sm_100
    d |= (uint64_t)layout_type << 61;
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

// The same with the accumulate flag known at compile time: no register, no compare.
template <bool ACCUMULATE>
__device__ __forceinline__ void umma_s8_c(
        uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
    asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "n"(ACCUMULATE ? 1 : 0)
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


// 16 columns, WITHOUT waiting: the registers may be read only after tmem_ld_wait16(v)
__device__ __forceinline__ void tmem_ld16_nowait(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
              "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]),
              "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
            : "r"(taddr)
            : "memory");
}

// Waits for this thread's TMEM loads. The registers are named as in/out operands so that
// the compiler cannot move a use of them above the wait.
__device__ __forceinline__ void tmem_ld_wait16(uint32_t (&v)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]),
                   "+r"(v[6]), "+r"(v[7]), "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]),
                   "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15])
                 :
                 : "memory");
}

__device__ __forceinline__ uint32_t pack4_prmt(int a, int b, int c, int d) {
    const uint32_t ab = __byte_perm((uint32_t)a, (uint32_t)b, 0x0040);
    const uint32_t cd = __byte_perm((uint32_t)c, (uint32_t)d, 0x0040);
    return __byte_perm(ab, cd, 0x5410);
}

// driver entry points for tensor-map encoding, resolved once at run time
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

inline const DriverApi& driver_api() {
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

inline int sm_count() {
    static int sms[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64)
        return 148;
    if (!sms[dev]) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
            v = 148;
        sms[dev] = v;
    }
    return sms[dev];
}

// CTAs of `threads` threads that one SM holds at once, from the kernel's register count,
// its dynamic shared memory and its TMEM columns. (The runtime's occupancy query answers 1
// for these kernels whatever their footprint, so the arithmetic is done here.)
template <class Kernel>
inline int resident_ctas_per_sm(Kernel kernel, int threads, int dynamic_smem, int tmem_cols) {
    cudaFuncAttributes fa;
    int regs = 128;
    if (cudaFuncGetAttributes(&fa, kernel) == cudaSuccess && fa.numRegs > 0)
        regs = fa.numRegs;
    const int regs_per_warp = (regs * 32 + 511) / 512 * 512;  // allocation granularity
    const int warps = (threads + 31) / 32;
    int by_regs = 65536 / (regs_per_warp * warps);
    int by_smem = (227 * 1024) / (dynamic_smem + 1024);
    int by_tmem = tmem_cols > 0 ? 512 / tmem_cols : 32;
    int n = by_regs < by_smem ? by_regs : by_smem;
    n = n < by_tmem ? n : by_tmem;
    return n < 1 ? 1 : n;
}

}  // namespace umma
}  // namespace mb200
