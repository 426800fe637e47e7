// Measures what the tensor pipe sustains on this GPU for tcgen05.mma kind::i8 (and kind::tf32):
// one CTA per SM issues a long run of 128 x 256 x (32 bytes of K) MMAs on operand tiles that
// already sit in shared memory (pseudo-random bytes, 128-byte swizzle, the same descriptors the
// ConvBias kernels use), so nothing but the MMA issue and the operand reads from shared memory
// limits it. The figure is the roofline denominator the benchmark reports fractions against
// when no int8 / tf32 peak has been measured for the pool.
#include "../../include/megcc_b200.h"
#include "internal.h"
#include "umma_ptx.cuh"

namespace mb200 {

using namespace umma;

namespace {

constexpr int kRateN = 256;
constexpr int kTileBytes = 128 * 128 + kRateN * 128;  // A 128 rows, B 256 rows of 128 bytes

template <bool TF32>
__global__ void __launch_bounds__(128, 1) mma_rate_kernel(int iters, int* status) {
    extern __shared__ uint8_t raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t bar;
    __shared__ uint32_t slot;
    __shared__ int abort_flag;
    // small finite values in either interpretation (int8 bytes; floats near 1.0)
    for (int i = threadIdx.x; i < kTileBytes / 4; i += blockDim.x)
        ((uint32_t*)smem)[i] = TF32 ? (0x3F800000u | ((0x9E3779B9u * (i + 1)) & 0x007FE000u))
                                    : 0x9E3779B9u * (i + 1);
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                             smem_u32(&slot)),
                     "r"(kRateN)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = slot;
    if (threadIdx.x == 0) {
        const uint32_t idesc = TF32 ? ((1u << 4) | (2u << 7) | (2u << 10) |
                                       ((uint32_t)(kRateN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24))
                                    : umma_idesc_s8(128, kRateN);
        const uint64_t a0 = umma_smem_desc(smem_u32(smem), 16, 1024, 2);
        const uint64_t b0 = umma_smem_desc(smem_u32(smem) + 128 * 128, 16, 1024, 2);
        for (int i = 0; i < iters; ++i) {
            // four K steps of 32 bytes walk the 128-byte row, as in the ConvBias main loop
            const uint64_t step = (uint64_t)((i & 3) * 2);
            const char* kind_unused = nullptr;
            (void)kind_unused;
            if (TF32)
                asm volatile(
                        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem),
                        "l"(a0 + step), "l"(b0 + step), "r"(idesc), "r"(i ? 1u : 0u)
                        : "memory");
            else
                umma_s8(tmem, a0 + step, b0 + step, idesc, i ? 1u : 0u);
        }
        umma_commit(&bar);
        if (!mbar_wait(&bar, 0, &abort_flag))
            atomicExch(status, ERR_DRAIN_WAIT);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x < 32)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem),
                     "r"(kRateN)
                     : "memory");
}

}  // namespace

}  // namespace mb200

using namespace mb200;

extern "C" int mb200_measure_mma_rate(int kind, void* stream, double* tera_ops_per_second) {
    if (!tera_ops_per_second || (kind != 0 && kind != 1))
        return set_error(ST_NULL_PTR, "measure_mma_rate: kind 0 (i8) or 1 (tf32) and a result pointer");
    cudaStream_t st = (cudaStream_t)stream;
    int* status = device_status_word(st);
    if (!status)
        return ST_MALLOC;
    const int smem = kTileBytes + 1024;
    auto kernel = kind == 0 ? mma_rate_kernel<false> : mma_rate_kernel<true>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return check_launch("mma_rate smem attribute");
    const int grid = umma::sm_count();
    const int iters = 40000;
    cudaEvent_t e0, e1;
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess)
        return check_launch("mma_rate events");
    kernel<<<grid, 128, smem, st>>>(2000, status);  // warm-up
    cudaEventRecord(e0, st);
    kernel<<<grid, 128, smem, st>>>(iters, status);
    cudaEventRecord(e1, st);
    int rc = check_launch("mma_rate");
    float ms = 0.f;
    if (!rc && (cudaEventSynchronize(e1) != cudaSuccess ||
                cudaEventElapsedTime(&ms, e0, e1) != cudaSuccess))
        rc = check_launch("mma_rate timing");
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (rc)
        return rc;
    // 2 * M * N * K operations per MMA; K = 32 int8 or 8 tf32 values (32 bytes either way)
    const double k = kind == 0 ? 32.0 : 8.0;
    *tera_ops_per_second = (double)grid * iters * 2.0 * 128.0 * kRateN * k / (ms * 1e-3) / 1e12;
    return ST_SUCCESS;
}
