// qint8 ConvBias for wide layers: implicit GEMM on a PAIR of SMs (tcgen05 cta_group::2).
//
// The im2col kernel of conv_umma.cu is limited by how fast operands arrive from L2: about
// 190 KB can be in flight per SM and a TMA load takes some 2000 cycles under load, i.e.
// roughly 60-80 bytes per clock and SM, while a 128 x 256 tile consumes 48 KB per 512 MMA
// cycles (94 B/clk). Here two CTAs of a cluster, one per SM, compute one 256 (pixels) x 256
// (output channels) tile: each loads its own 128 pixels of A and ONE HALF of the filter
// tile, and a single thread of the leader CTA issues M = 256 MMAs that read both halves.
// Per SM that is 32 KB per 512 MMA cycles (64 B/clk) and six 32 KB stages in flight.
//
//   both CTAs : warp 0 = TMA producer (own A tile, own half of B; completion is counted on
//               the LEADER's full barrier), warps 2..17 = epilogue of the own 128 TMEM lanes
//   leader    : warp 1 = MMA issuer; its commits arrive on the empty / accumulator-full
//               barriers of both CTAs (two commits, no multicast form)
//   peer      : epilogue warps release the accumulator on the leader's barrier (remote arrive)
//
// Every wait is bounded as in conv_umma.cu; a CTA that gives up also raises its peer's abort
// flag. No load uses cluster multicast.
#include <stdio.h>
#include <stdlib.h>

#include "conv_epilogue.cuh"
#include "internal.h"
#include "tuning.h"
#include "umma_ptx.cuh"

namespace mb200 {

using namespace umma;

namespace {

constexpr int kBM = 128;   // pixels per CTA (the pair covers 256)
constexpr int kBN = 256;   // output channels per tile
constexpr int kBNh = 128;  // filter rows each CTA loads
constexpr int kBK = 128;   // K bytes per stage (128-byte swizzle rows)
constexpr int kSt = 6;
constexpr int kEpilogueWarps = 16;
constexpr int kThreads = 64 + 32 * kEpilogueWarps;
constexpr int kABytes = kBM * kBK, kBBytes = kBNh * kBK;
constexpr int kBarOff = kSt * (kABytes + kBBytes);
constexpr int kDynamic = kBarOff + (2 * kSt + 5) * 8 + 16 + 1024;

struct PairParams {
    int m_total, oc, oh, ow;
    int cblocks, taps_w, k_iters;
    int sh, sw, base_h, base_w, dh, dw;
    int m_tiles, n_tiles;  // in pair tiles: 256 pixels x 256 channels
    EpilogueParams ep;
    int8_t* dst;
    int* status;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t num_clusters_x() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
    return r;
}
// the shared::cluster address of `local` (an address in this CTA's shared memory) in CTA `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity), "r"(2000u)
            : "memory");
    return ok != 0;
}
// bounded wait on a barrier that the other CTA of the pair (or a commit issued there) arrives on
__device__ __forceinline__ bool mbar_wait_cluster(
        uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
        if (mbar_try_wait_cluster(bar, parity))
            return true;
    const long long t0 = clock64();
    for (int spin = 0;; ++spin) {
        if (mbar_try_wait_cluster(bar, parity))
            return true;
        if (spin > 256)
            __nanosleep(128);
        if ((spin & 63) == 63) {
            if (*abort_flag)
                return false;
            if (clock64() - t0 > kWaitCycles)
                return false;
        }
    }
}
// TMA loads of a CTA pair: the data lands in THIS CTA's shared memory, the byte count is
// reported to the barrier at `mbar_cluster_addr`, which may belong to the other CTA
__device__ __forceinline__ void tma_pair_load_2d(
        void* smem, const CUtensorMap* map, uint32_t mbar_cluster_addr, int c0, int c1) {
    asm volatile(
            "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem)),
            "l"((uint64_t)map), "r"(mbar_cluster_addr), "r"(c0), "r"(c1)
            : "memory");
}
__device__ __forceinline__ void tma_pair_load_im2col_4d(
        void* smem, const CUtensorMap* map, uint32_t mbar_cluster_addr, int c, int w, int h, int n,
        uint16_t off_w, uint16_t off_h) {
    asm volatile(
            "cp.async.bulk.tensor.4d.im2col.cta_group::2.shared::cluster.global"
            ".mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};" ::"r"(
                    smem_u32(smem)),
            "l"((uint64_t)map), "r"(mbar_cluster_addr), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w),
            "h"(off_h)
            : "memory");
}
__device__ __forceinline__ void umma_pair_s8(
        uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
}
// arrives (once) on the barrier at a shared::cluster address when the pair's MMAs issued so
// far have retired
__device__ __forceinline__ void umma_pair_commit(uint32_t bar_cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                         bar_cluster_addr)
                 : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1) conv_pair_kernel(
        const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
        const PairParams p) {
    extern __shared__ uint8_t smem_raw[];
    // the dynamic window starts at the same offset in both CTAs, so the aligned pointers,
    // and with them every barrier and tile offset, agree between the two
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* tiles_a = smem;
    uint8_t* tiles_b = smem + kSt * kABytes;
    uint64_t* full_bar = (uint64_t*)(smem + kBarOff);  // used in the leader only
    uint64_t* empty_bar = full_bar + kSt;              // one set per CTA
    uint64_t* acc_full = empty_bar + kSt;              // [2], one set per CTA
    uint64_t* acc_empty = acc_full + 2;                // [2], used in the leader only
    uint64_t* drain_bar = acc_empty + 2;
    uint32_t* tmem_slot = (uint32_t*)(drain_bar + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int total_tiles = p.m_tiles * p.n_tiles;
    const int first_tile = (int)cluster_id_x(), tile_step = (int)num_clusters_x();

    if (threadIdx.x == 0) {
        for (int s = 0; s < kSt; ++s) {
            mbar_init(&full_bar[s], 1);   // the leader's producer; both CTAs' bytes
            mbar_init(&empty_bar[s], 1);  // one commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 2 * kEpilogueWarps);  // one arrival per epilogue warp
        }
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        // the same warp of both CTAs allocates the pair's columns
        asm volatile(
                "tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                        smem_u32(tmem_slot)),
                "r"(2 * kBN)
                : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync();  // both CTAs' barriers exist before anything arrives on them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t peer_abort = map_to_cta(smem_u32((const void*)abort_flag), rank ^ 1u);

    // gives up: records the code, stops the own roles and tells the other CTA
    auto give_up = [&](int code) {
        if (!*abort_flag) {
            *abort_flag = 1;
            atomicExch(p.status, code);
        }
        asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(peer_abort), "r"(1) : "memory");
    };

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (lane == 0) {
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step) {
                const int tile_n = tile % p.n_tiles, tile_m = tile / p.n_tiles;
                const int m0 = tile_m * (2 * kBM) + (int)rank * kBM;
                const int n0 = tile_n * kBN + (int)rank * kBNh;
                const int img = m0 / (p.oh * p.ow);
                const int rem = m0 - img * (p.oh * p.ow);
                const int oy = rem / p.ow, ox = rem - oy * p.ow;
                const int base_w = ox * p.sw + p.base_w, base_h = oy * p.sh + p.base_h;
                int cb = 0, fx = 0, fy = 0;
                for (int it = 0; it < p.k_iters; ++it) {
                    if (!mbar_wait_cluster(&empty_bar[s], phase ^ 1u, abort_flag)) {
                        give_up(ERR_PRODUCER_WAIT);
                        ok = false;
                        break;
                    }
                    const uint32_t full_leader = map_to_cta(smem_u32(&full_bar[s]), 0);
                    if (leader)
                        mbar_expect_tx(&full_bar[s], 2u * (uint32_t)(kABytes + kBBytes));
                    tma_pair_load_im2col_4d(tiles_a + s * kABytes, &map_a, full_leader, cb * kBK,
                                            base_w, base_h, img, (uint16_t)(fx * p.dw),
                                            (uint16_t)(fy * p.dh));
                    tma_pair_load_2d(tiles_b + s * kBBytes, &map_b, full_leader, it * kBK, n0);
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
        // ---------------- MMA issuer (leader only) ----------------
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = umma_idesc_s8(2 * kBM, kBN);
            int local = 0, s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step, ++local) {
                const int buf = local & 1;
                const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
                // both CTAs' epilogues must have drained this accumulator buffer
                if (!mbar_wait_cluster(&acc_empty[buf], acc_phase ^ 1u, abort_flag)) {
                    give_up(ERR_MMA_ACC_WAIT);
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + (uint32_t)(buf * kBN);
                for (int it = 0; it < p.k_iters; ++it) {
                    if (!mbar_wait_cluster(&full_bar[s], phase, abort_flag)) {
                        give_up(ERR_MMA_WAIT);
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    // offsets inside the CTA's window: the same in both CTAs of the pair
                    const uint64_t adesc =
                            umma_smem_desc(smem_u32(tiles_a + s * kABytes), 16, 1024, 2);
                    const uint64_t bdesc =
                            umma_smem_desc(smem_u32(tiles_b + s * kBBytes), 16, 1024, 2);
#pragma unroll
                    for (int k = 0; k < kBK / 32; ++k)
                        umma_pair_s8(tmem_d, adesc + k * 2, bdesc + k * 2, idesc,
                                     (it | k) != 0 ? 1u : 0u);
                    // the stage is free in both CTAs once these MMAs retire
                    const uint32_t e_local = smem_u32(&empty_bar[s]);
                    umma_pair_commit(e_local);
                    umma_pair_commit(map_to_cta(e_local, 1));
                    if (++s == kSt) {
                        s = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) {
                    const uint32_t f_local = smem_u32(&acc_full[buf]);
                    umma_pair_commit(f_local);
                    umma_pair_commit(map_to_cta(f_local, 1));
                }
            }
        }
    } else {
        // ---------------- epilogue (both CTAs): warps 2..17, TMEM lanes 32*(warp%4).. -------
        const int q = warp & 3;
        const int row = q * 32 + lane;
        int local = 0;
        bool ok = true;
        for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step, ++local) {
            const int buf = local & 1;
            const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
            const int tile_n = tile % p.n_tiles, tile_m = tile / p.n_tiles;
            const int m = tile_m * (2 * kBM) + (int)rank * kBM + row, n0 = tile_n * kBN;
            ok = mbar_wait_cluster(&acc_full[buf], acc_phase, abort_flag);
            if (!ok)
                give_up(ERR_EPILOGUE_WAIT);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * kBN);
            const int first = (warp - 2) >> 2;
            // each warp takes a run of adjacent chunks: its thread's bytes are contiguous
            constexpr int kChunksPerWarp = (kBN / 32) / (kEpilogueWarps / 4);
#pragma unroll 1
            for (int c = first * kChunksPerWarp; c < (first + 1) * kChunksPerWarp; ++c) {
                uint32_t v[32];
                tmem_ld32(taddr + (uint32_t)(c * 32), v);
                if (c + 1 == (first + 1) * kChunksPerWarp) {
                    // this warp's accumulators are in registers: release the buffer (one
                    // arrival per warp, on the leader's barrier)
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0)
                        mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
                }
                const int ch0 = n0 + c * 32;
                if (m < p.m_total && ch0 < p.oc)
                    epilogue_store<32>(v, p.ep, p.dst, (size_t)m * p.oc + ch0, ch0);
            }
        }
    }

    // ---------------- teardown ----------------
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_flag) {
        // a wait ran out: let loads in flight land and MMAs retire (both bounded) before
        // the shared memory and TMEM are given back
        if (warp == 1 && lane == 0 && leader) {
            umma_pair_commit(smem_u32(drain_bar));
            const long long t0 = clock64();
            while (!mbar_try_wait_cluster(drain_bar, 0)) {
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
    // neither CTA may leave (or free TMEM) while the other can still reach its barriers,
    // its shared memory or its accumulators
    cluster_sync();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(2 * kBN)
                     : "memory");
    }
}

}  // namespace

bool conv_pair_supported(
        const ConvArgs& a, const int8_t* src, const int8_t* flt, const int8_t* dst) {
    // im2col maps only: the small-tensor limit of conv_umma.cu applies to every shape here
    return conv_umma_supported(a, src, flt, dst) && a.ic % kBK == 0 && a.oc > kBNh &&
           (size_t)a.n * a.ih * a.iw * a.ic >= 131072;
}

// Clusters of this kernel that the GPU holds at once (one CTA per SM, so at most half the SM
// count), as the occupancy query sees it.
static int pair_clusters_resident() {
    static int cached[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64)
        return sm_count() / 2;
    if (!cached[dev]) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * (sm_count() / 2), 1, 1);
        cfg.blockDim = dim3(kThreads, 1, 1);
        cfg.dynamicSmemBytes = kDynamic;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, conv_pair_kernel, &cfg) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = sm_count() / 2;
        }
        if (n > sm_count() / 2)
            n = sm_count() / 2;
        cached[dev] = n;
    }
    return cached[dev];
}

// `a`: dense convolution over an NHWC source with ic % 128 == 0; filter [OC][KH][KW][IC].
int launch_conv_pair(
        const ConvArgs& a, const int8_t* src, const int8_t* flt, const int32_t* bias,
        const float* flt_scales, int8_t* dst, cudaStream_t st) {
    const DriverApi& api = driver_api();
    if (!api.ok)
        return set_error(ST_RUNTIME, "cuTensorMapEncode* entry points not found in the driver");
    if (((uintptr_t)bias & 15) || ((uintptr_t)flt_scales & 15))
        return set_error(ST_INVALID_LAYOUT, "bias and channel scales must be 16-byte aligned");
    const int taps = a.kh * a.kw;
    CUtensorMap map_a, map_b;
    {
        cuuint64_t dims[4] = {(cuuint64_t)a.ic, (cuuint64_t)a.iw, (cuuint64_t)a.ih,
                              (cuuint64_t)a.n};
        cuuint64_t strides[3] = {(cuuint64_t)a.ic, (cuuint64_t)a.iw * a.ic,
                                 (cuuint64_t)a.ih * a.iw * a.ic};
        // bounding box of the first-tap positions: from -pad to the last output's position
        int lower[2] = {-a.pw, -a.ph};
        int upper[2] = {(a.ow - 1) * a.sw - a.pw - (a.iw - 1), (a.oh - 1) * a.sh - a.ph - (a.ih - 1)};
        cuuint32_t estr[4] = {1, (cuuint32_t)a.sw, (cuuint32_t)a.sh, 1};
        CUresult r = api.im2col(
                &map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)src, dims, strides, lower, upper,
                kBK, kBM, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return set_error(ST_RUNTIME, "cuTensorMapEncodeIm2col failed: %d", (int)r);
    }
    {
        const cuuint64_t k_total = (cuuint64_t)taps * a.ic;
        cuuint64_t dims[2] = {k_total, (cuuint64_t)a.oc};
        cuuint64_t strides[1] = {k_total};
        cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)kBNh};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = api.tiled(
                &map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)flt, dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return set_error(ST_RUNTIME, "cuTensorMapEncodeTiled failed: %d", (int)r);
    }

    PairParams p;
    p.m_total = a.m;
    p.oc = a.oc;
    p.oh = a.oh;
    p.ow = a.ow;
    p.cblocks = a.ic / kBK;
    p.taps_w = a.kw;
    p.k_iters = taps * p.cblocks;
    p.sh = a.sh;
    p.sw = a.sw;
    p.base_h = -a.ph;
    p.base_w = -a.pw;
    p.dh = a.dh;
    p.dw = a.dw;
    p.m_tiles = (a.m + 2 * kBM - 1) / (2 * kBM);
    p.n_tiles = (a.oc + kBN - 1) / kBN;
    p.ep.oc = a.oc;
    p.ep.act = a.act;
    p.ep.bounded = requant_is_bounded(a.s_src, a.s_flt, a.s_dst) ? 1 : 0;
    p.ep.s_src = a.s_src;
    p.ep.s_flt = a.s_flt;
    p.ep.s_dst = a.s_dst;
    p.ep.inv_dst = 1.0f / a.s_dst;  // correctly rounded on the host
    // a fused step follows a ConvBias without activation
    p.ep.fast_mul = p.ep.fast_add = 0.f;
    p.ep.fast_ops = 0;
    if (p.ep.bounded && !flt_scales)
        p.ep.fast_ops = requant_fast_constants(a.s_src, a.s_flt, a.s_dst,
                                               (a.z && a.z_mode) ? ACT_IDENTITY : a.act,
                                               &p.ep.fast_mul, &p.ep.fast_add);
    p.ep.bias = bias;
    p.ep.flt_scales = flt_scales;
    p.ep.z = a.z;
    p.ep.z_mode = a.z ? a.z_mode : 0;
    p.ep.z_scale = a.z_scale;
    p.ep.z_div = 1.0f / a.z_out_scale;  // the reference's scale_div = 1.f / scale_dst
    p.ep.z_fast_a = p.ep.z_fast_b = 0.f;
    if (p.ep.z_mode != 0 && p.ep.fast_ops != 0)
        residual_fast_constants(a.s_dst, a.z_scale, a.z_out_scale, p.ep.z_mode, &p.ep.z_fast_a,
                                &p.ep.z_fast_b);
    p.ep.acc_out = a.acc_out;
    p.dst = dst;
    p.status = device_status_word(st);
    if (!p.status)
        return ST_MALLOC;
    if (cudaFuncSetAttribute(conv_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kDynamic) != cudaSuccess)
        return check_launch("conv_pair smem attribute");
    const int total = p.m_tiles * p.n_tiles;
    int clusters = pair_clusters_resident();
    if (clusters > total)
        clusters = total;
    if (tuning().debug)
        fprintf(stderr, "conv_pair: clusters %d tiles %d k_iters %d smem %d\n", clusters, total,
                p.k_iters, kDynamic);
    conv_pair_kernel<<<2 * clusters, kThreads, kDynamic, st>>>(map_a, map_b, p);
    return check_launch("conv_pair");
}

}  // namespace mb200
