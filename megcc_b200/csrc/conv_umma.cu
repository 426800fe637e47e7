// qint8 ConvBias as implicit GEMM on the sm_100a tensor cores.
//
//   D[m, oc] = sum_{fy,fx,c} A[m, (fy,fx,c)] * W[oc, (fy,fx,c)],   m = (n, oh, ow) linearised
//
// * activations NHWC int8. One TMA im2col load brings, for one filter tap, the channels of
//   the 128 consecutive output pixels of a tile straight into a K-major shared-memory tile;
//   padding and stride are resolved by the im2col bounding box and traversal stride.
// * filter pre-packed K-major [OC][taps][channels], fetched by tiled 2D TMA.
// * tcgen05.mma kind::i8, M=128 x N=BN x K=32 per instruction, int32 accumulators in TMEM,
//   two accumulator buffers so the epilogue of one tile overlaps the MMAs of the next.
// * persistent CTAs walk the tile list; warp 0 = TMA producer, warp 1 = MMA issuer (+ TMEM
//   alloc), warps 2..9 = epilogue (tcgen05.ld -> +bias -> fp32 requantisation in the
//   reference's operation order -> activation -> int8 -> 16-byte stores).
// * every wait is bounded: when it runs out the kernel records a code in the device status
//   word, drains what it started, frees its TMEM and returns.
//
// Two operand geometries:
//   WIDE  one tap x 64 channels per pipeline stage, 64-byte swizzle (input channels % 64 == 0)
//   TAP16 four taps x 16 channels per stage, no swizzle: the form a stride-2 convolution with
//         at most 4 input channels takes after a 2x2 space-to-depth step (see conv_s2d.cu)
//
// Replaces the loop nest of compiler/lib/KernelGen/BareMetal/ConvKernel.cpp:305-344 and
// its epilogue (:374-382, BareMetal/Activation.cpp:105-113).
#include <stdio.h>
#include <stdlib.h>

#include <map>
#include <mutex>
#include <utility>

#include "conv_epilogue.cuh"
#include "internal.h"
#include "pdl.h"
#include "tuning.h"
#include "umma_ptx.cuh"

namespace mb200 {

using namespace umma;

namespace {

constexpr int kBM = 128;     // output pixels per tile (UMMA M)
constexpr int kBK = 64;      // K bytes per pipeline stage of the 64-byte geometries
constexpr int kUmmaK = 32;   // K per tcgen05.mma kind::i8
constexpr int kStages = 6;         // most stages any variant uses (sizes the barrier arrays)
enum Geometry : int { GEOM_WIDE = 0, GEOM_TAP16 = 1, GEOM_WIDE128 = 2 };

// Per output-channel tile width. BN = 64 / 128: two accumulator buffers of BN columns, up
// to three CTAs per SM, two epilogue warps per TMEM lane quarter. BN = 256 (only with
// 128-byte rows): the two buffers fill the SM's 512 TMEM columns, so one CTA per SM, which
// then gets four epilogue warps per lane quarter and a larger register budget. The wide
// tile exists because the operands come from L2 at well under 100 bytes per clock and SM:
// a 128 x 128 tile needs 32 KB per 256 MMA cycles, a 128 x 256 tile 48 KB per 512.
template <int BN>
struct Shape {
    static constexpr int kEpilogueWarps = BN == 256 ? 16 : 8;
    static constexpr int kEpilogueThreads = 32 * kEpilogueWarps;
    static constexpr int kThreads = 64 + kEpilogueThreads;
    static constexpr int kMinCtas = BN == 256 ? 1 : 2;
};

// K bytes and pipeline depth per geometry. WIDE128 moves 128-channel rows (128-byte swizzle):
// half as many TMA requests and barrier round trips per byte as WIDE.
template <int BN, int GEOM>
struct Geom {
    static constexpr int kBKg = GEOM == GEOM_WIDE128 ? 128 : 64;
    static constexpr int kStagesG = GEOM == GEOM_WIDE128 ? (BN == 256 ? 4 : 3) : kStages;
};

struct UmmaConvParams {
    int m_total, oc, oh, ow;
    int cblocks;        // WIDE: 64-channel blocks per tap
    int taps_w;         // filter taps along W (TAP16: taps of the space-to-depth filter)
    int k_iters;        // pipeline stages per tile
    int sh, sw;         // output -> base pixel scaling
    int base_h, base_w; // coordinate of output (0,0)'s first tap (= -pad)
    int dh, dw;
    int m_tiles, n_tiles;
    int a_tiled;        // 1x1, stride 1, no padding: A is the plain matrix [pixels][channels]
    EpilogueParams ep;
    int8_t* dst;
    int* status;
    // cycles a bounded wait may take (kWaitCycles unless a self-test shortens it), and the
    // pipeline step of every tile that the producer leaves out (-1: none; self-test only)
    long long wait_cycles;
    int skip_step;
    // split-K (SPLITK kernels only): work items below `full_tiles` are whole tiles, the
    // tiles after them are cut into `split` parts of `k_per_part` pipeline steps each
    int full_tiles, split, k_per_part, total_items;
    int overlap;          // 1: chunks of the verified short forms load their accumulators in two halves
    int4* slabs;          // [split item][chunk][16-byte group][row]: one part's accumulators
    unsigned* counters;   // [split tile] parts finished; zero between launches
};

// One unit of work of a persistent CTA: a whole tile, or one K range of a split tile.
struct WorkItem {
    int tile, k0, k1;
    int slot;  // index of the split item (its slab), -1 for a whole tile
};

template <bool SPLITK>
__device__ __forceinline__ WorkItem decode_item(const UmmaConvParams& p, int item) {
    WorkItem w;
    if (!SPLITK || item < p.full_tiles) {
        w.tile = item;
        w.k0 = 0;
        w.k1 = p.k_iters;
        w.slot = -1;
    } else {
        const int idx = item - p.full_tiles;
        const int t = idx / p.split, part = idx - t * p.split;
        w.tile = p.full_tiles + t;
        w.k0 = part * p.k_per_part;
        w.k1 = min(w.k0 + p.k_per_part, p.k_iters);
        w.slot = idx;
    }
    return w;
}

template <int BN, int GEOM>
struct SmemLayout {
    static constexpr int kABytes = kBM * Geom<BN, GEOM>::kBKg;
    static constexpr int kBBytes = BN * Geom<BN, GEOM>::kBKg;
    static constexpr int kTiles = Geom<BN, GEOM>::kStagesG * (kABytes + kBBytes);
    // after the tiles: full[kStages], empty[kStages], acc_full[2], acc_empty[2], drain,
    // the epilogue's own rendezvous (split-K), then three words
    static constexpr int kBarOff = kTiles;
    static constexpr int kTotal = kBarOff + (2 * kStages + 6) * 8 + 16;
    static constexpr int kDynamic = kTotal + 1024;  // room to align the tiles to 1024 bytes
};

template <int BN, int GEOM, bool SPLITK = false>
__global__ void __launch_bounds__(Shape<BN>::kThreads, Shape<BN>::kMinCtas) conv_umma_kernel(
        const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
        const UmmaConvParams p) {
    using L = SmemLayout<BN, GEOM>;
    constexpr int kBKc = Geom<BN, GEOM>::kBKg;
    constexpr int kSt = Geom<BN, GEOM>::kStagesG;
    constexpr int kEpilogueWarps = Shape<BN>::kEpilogueWarps;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* tiles_a = smem;
    uint8_t* tiles_b = smem + kSt * L::kABytes;
    uint64_t* full_bar = (uint64_t*)(smem + L::kBarOff);
    uint64_t* empty_bar = full_bar + kStages;
    uint64_t* acc_full = empty_bar + kStages;  // [2]
    uint64_t* acc_empty = acc_full + 2;        // [2]
    uint64_t* drain_bar = acc_empty + 2;
    uint64_t* ep_bar = drain_bar + 1;
    uint32_t* tmem_slot = (uint32_t*)(ep_bar + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    volatile int* last_flag = (volatile int*)(tmem_slot + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_tiles = SPLITK ? p.total_items : p.m_tiles * p.n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 32 * kEpilogueWarps);  // every epilogue thread arrives
        }
        mbar_init(drain_bar, 1);
        mbar_init(ep_bar, 32 * kEpilogueWarps);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile(
                "tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                        smem_u32(tmem_slot)),
                "r"(2 * BN)
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
            // this thread runs alone in its warp and every instruction costs it several
            // cycles: stage, phase and filter tap are running counters, no division per step
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < total_tiles && ok; item += gridDim.x) {
                const WorkItem w = decode_item<SPLITK>(p, item);
                const int tile = w.tile;
                const int tile_n = tile % p.n_tiles, tile_m = tile / p.n_tiles;
                const int m0 = tile_m * kBM, n0 = tile_n * BN;
                const int img = m0 / (p.oh * p.ow);
                const int rem = m0 - img * (p.oh * p.ow);
                const int oy = rem / p.ow, ox = rem - oy * p.ow;
                const int base_w = ox * p.sw + p.base_w, base_h = oy * p.sh + p.base_h;
                int cb = 0, fx = 0, fy = 0;
                if (SPLITK && w.k0 != 0) {
                    // a later part of a split tile starts in the middle of the filter
                    cb = w.k0 % p.cblocks;
                    const int tap = w.k0 / p.cblocks;
                    fy = tap / p.taps_w;
                    fx = tap - fy * p.taps_w;
                }
                for (int it = w.k0; it < w.k1; ++it) {
                    if (!mbar_wait(&empty_bar[s], phase ^ 1u, abort_flag, p.wait_cycles)) {
                        if (!*abort_flag) {
                            *abort_flag = 1;
                            atomicExch(p.status, ERR_PRODUCER_WAIT);
                        }
                        ok = false;
                        break;
                    }
                    if (it == p.skip_step) {
                        // self-test of the bounded waits: this stage is never filled (neither
                        // the byte count is announced nor a load issued), so the MMA thread's
                        // wait for it runs out and the kernel takes its give-up path
                        if (++s == kSt) {
                            s = 0;
                            phase ^= 1u;
                        }
                        continue;
                    }
                    mbar_expect_tx(&full_bar[s], (uint32_t)(L::kABytes + L::kBBytes));
                    uint8_t* sa = tiles_a + s * L::kABytes;
                    uint8_t* sb = tiles_b + s * L::kBBytes;
                    if (GEOM != GEOM_TAP16) {
                        if (p.a_tiled)
                            tma_load_2d(sa, &map_a, &full_bar[s], cb * kBKc, m0);
                        else
                            tma_load_im2col_4d(sa, &map_a, &full_bar[s], cb * kBKc, base_w, base_h,
                                               img, (uint16_t)(fx * p.dw), (uint16_t)(fy * p.dh));
                        tma_load_2d(sb, &map_b, &full_bar[s], it * kBKc, n0);
                        if (++cb == p.cblocks) {
                            cb = 0;
                            if (++fx == p.taps_w) {
                                fx = 0;
                                ++fy;
                            }
                        }
                    } else {
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            tma_load_im2col_4d(sa + t * (kBM * 16), &map_a, &full_bar[s], 0, base_w,
                                               base_h, img, (uint16_t)fx, (uint16_t)fy);
                            tma_load_2d(sb + t * (BN * 16), &map_b, &full_bar[s], (it * 4 + t) * 16,
                                        n0);
                            if (++fx == p.taps_w) {
                                fx = 0;
                                ++fy;
                            }
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
            constexpr uint32_t idesc = umma_idesc_s8(kBM, BN);
            int local = 0, s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < total_tiles && ok; item += gridDim.x, ++local) {
                const WorkItem w = decode_item<SPLITK>(p, item);
                const int buf = local & 1;
                const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
                // the epilogue must have drained this accumulator buffer
                if (!mbar_wait(&acc_empty[buf], acc_phase ^ 1u, abort_flag, p.wait_cycles)) {
                    if (!*abort_flag) {
                        *abort_flag = 1;
                        atomicExch(p.status, ERR_MMA_ACC_WAIT);
                    }
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
                for (int it = w.k0; it < w.k1; ++it) {
                    if (!mbar_wait(&full_bar[s], phase, abort_flag, p.wait_cycles)) {
                        if (!*abort_flag) {
                            *abort_flag = 1;
                            atomicExch(p.status, ERR_MMA_WAIT);
                        }
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_u32(tiles_a + s * L::kABytes);
                    const uint32_t b_addr = smem_u32(tiles_b + s * L::kBBytes);
                    // one descriptor per operand and stage; a K step only moves the address
                    // field (16-byte units): +32 bytes inside the swizzled row, or two 16-byte
                    // tap blocks in the plain layout
                    uint64_t adesc, bdesc;
                    uint32_t a_step, b_step;
                    if (GEOM == GEOM_WIDE128) {
                        // 128-byte swizzle: 8-row groups 1024 bytes apart
                        adesc = umma_smem_desc(a_addr, 16, 1024, 2);
                        bdesc = umma_smem_desc(b_addr, 16, 1024, 2);
                        a_step = b_step = 32 / 16;
                    } else if (GEOM == GEOM_WIDE) {
                        adesc = umma_smem_desc(a_addr, 16, 512, 4);
                        bdesc = umma_smem_desc(b_addr, 16, 512, 4);
                        a_step = b_step = 32 / 16;
                    } else {
                        adesc = umma_smem_desc(a_addr, kBM * 16, 128, 0);
                        bdesc = umma_smem_desc(b_addr, BN * 16, 128, 0);
                        a_step = 2 * (kBM * 16) / 16;
                        b_step = 2 * (BN * 16) / 16;
                    }
                    umma_s8(tmem_d, adesc, bdesc, idesc, it != w.k0 ? 1u : 0u);
#pragma unroll
                    for (int k = 1; k < kBKc / kUmmaK; ++k)
                        umma_s8_c<true>(tmem_d, adesc + k * a_step, bdesc + k * b_step, idesc);
                    umma_commit(&empty_bar[s]);  // frees the stage once these MMAs retire
                    if (++s == kSt) {
                        s = 0;
                        phase ^= 1u;
                    }
                }
                if (ok)
                    umma_commit(&acc_full[buf]);
            }
        }
    } else {
        // ---------------- epilogue: warps 2..9, TMEM lanes 32*(warp%4).. ----------------
        const int q = warp & 3;
        const int row = q * 32 + lane;
        int local = 0;
        bool ok = true;
        uint32_t ep_phase = 0;  // parity of the epilogue's own rendezvous (split-K)
        const bool overlap_ok = p.overlap && epilogue_chunk_overlappable(p.ep, p.dst, 0);
        for (int item = blockIdx.x; item < total_tiles && ok; item += gridDim.x, ++local) {
            const WorkItem w = decode_item<SPLITK>(p, item);
            const int tile = w.tile;
            const int buf = local & 1;
            const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
            const int tile_n = tile % p.n_tiles, tile_m = tile / p.n_tiles;
            const int m = tile_m * kBM + row, n0 = tile_n * BN;
            ok = mbar_wait(&acc_full[buf], acc_phase, abort_flag, p.wait_cycles);
            if (!ok && !*abort_flag) {
                *abort_flag = 1;
                atomicExch(p.status, ERR_EPILOGUE_WAIT);
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
            const int half = (warp - 2) >> 2;
            // each warp takes a run of adjacent chunks: its thread's bytes are contiguous
            constexpr int kChunksPerWarp = (BN / 32) / (kEpilogueWarps / 4);
            static_assert(kChunksPerWarp >= 1, "every epilogue warp must own a chunk");
            if (SPLITK && w.slot >= 0) {
                // One K range of a split tile. Its raw accumulators go to this item's slab;
                // a slab is laid out [chunk][16-byte group][row], so a warp's 16-byte stores
                // (and the loads of the CTA that finishes the tile, whose threads own the same
                // rows and chunks) are 512 contiguous bytes. The CTA that finds the tile's
                // other parts already counted sums all slabs and requantises; nobody waits
                // for another CTA.
                constexpr int kSlabVecs = (BN / 32) * 8 * kBM;
                int4* slab = p.slabs + (size_t)w.slot * kSlabVecs;
#pragma unroll 1
                for (int c = half * kChunksPerWarp; c < (half + 1) * kChunksPerWarp; ++c) {
                    uint32_t v[32];
                    tmem_ld32(taddr + (uint32_t)(c * 32), v);
                    if (c + 1 == (half + 1) * kChunksPerWarp) {
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        mbar_arrive(&acc_empty[buf]);
                    }
#pragma unroll
                    for (int k = 0; k < 8; ++k)
                        __stcg(slab + (c * 8 + k) * kBM + row,
                               make_int4((int)v[4 * k], (int)v[4 * k + 1], (int)v[4 * k + 2],
                                         (int)v[4 * k + 3]));
                }
                __threadfence();  // the slab is visible device-wide before the part is counted
                mbar_arrive(ep_bar);
                ok = mbar_wait(ep_bar, ep_phase, abort_flag, p.wait_cycles);
                ep_phase ^= 1u;
                if (ok && threadIdx.x == 64) {
                    unsigned* counter = p.counters + (w.tile - p.full_tiles);
                    const unsigned before = atomicAdd(counter, 1u);
                    const bool last = before + 1u == (unsigned)p.split;
                    if (last)
                        *counter = 0;  // every part has been counted: ready for the next launch
                    *last_flag = last ? 1 : 0;
                }
                if (ok) {
                    mbar_arrive(ep_bar);
                    ok = mbar_wait(ep_bar, ep_phase, abort_flag, p.wait_cycles);
                    ep_phase ^= 1u;
                }
                if (!ok && !*abort_flag) {
                    *abort_flag = 1;
                    atomicExch(p.status, ERR_EPILOGUE_WAIT);
                }
                ok = __all_sync(0xffffffffu, ok);
                if (!ok)
                    break;
                if (*last_flag) {
                    __threadfence();
                    const int4* first = p.slabs + (size_t)(w.slot - w.slot % p.split) * kSlabVecs;
#pragma unroll 1
                    for (int c = half * kChunksPerWarp; c < (half + 1) * kChunksPerWarp; ++c) {
                        uint32_t v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            v[j] = 0;
                        for (int part = 0; part < p.split; ++part) {
                            const int4* s4 = first + (size_t)part * kSlabVecs + (c * 8) * kBM + row;
#pragma unroll
                            for (int k = 0; k < 8; ++k) {
                                const int4 t = __ldcg(s4 + k * kBM);
                                v[4 * k] += (uint32_t)t.x;
                                v[4 * k + 1] += (uint32_t)t.y;
                                v[4 * k + 2] += (uint32_t)t.z;
                                v[4 * k + 3] += (uint32_t)t.w;
                            }
                        }
                        const int ch0 = n0 + c * 32;
                        if (m < p.m_total && ch0 < p.oc)
                            epilogue_store<32>(v, p.ep, p.dst, (size_t)m * p.oc + ch0, ch0);
                    }
                }
                continue;
            }
#pragma unroll 1
            for (int c = half * kChunksPerWarp; c < (half + 1) * kChunksPerWarp; ++c) {
                if (overlap_ok && n0 + c * 32 + 32 <= p.oc) {
                    // a verified short form: the chunk's second 16 columns are fetched while
                    // the first are requantised (conv_epilogue.cuh)
                    const int ch0 = n0 + c * 32;
                    epilogue_chunk_overlapped(
                            taddr + (uint32_t)(c * 32), p.ep, p.dst, (size_t)m * p.oc + ch0, ch0,
                            m < p.m_total,
                            c + 1 == (half + 1) * kChunksPerWarp ? &acc_empty[buf] : nullptr);
                    continue;
                }
                uint32_t v[32];
                tmem_ld32(taddr + (uint32_t)(c * 32), v);
                if (c + 1 == (half + 1) * kChunksPerWarp) {
                    // all of this thread's accumulators are in registers: hand the buffer back
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    mbar_arrive(&acc_empty[buf]);
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
                     "r"(2 * BN)
                     : "memory");
    }
}

// ------------------------------------------------------------------------------------------
// host side: tensor maps and launch
// ------------------------------------------------------------------------------------------
template <int BN, int GEOM, bool SPLITK = false>
int launch_kernel(
        const CUtensorMap& ma, const CUtensorMap& mb, const UmmaConvParams& p, cudaStream_t st) {
    if (cudaFuncSetAttribute(
                conv_umma_kernel<BN, GEOM, SPLITK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                SmemLayout<BN, GEOM>::kDynamic) != cudaSuccess)
        return check_launch("conv_umma smem attribute");
    // persistent CTAs: as many as the SM holds at once
    constexpr int kThreads = Shape<BN>::kThreads;
    const int per_sm = resident_ctas_per_sm(
            conv_umma_kernel<BN, GEOM, SPLITK>, kThreads, SmemLayout<BN, GEOM>::kDynamic, 2 * BN);
    const int total = SPLITK ? p.total_items : p.m_tiles * p.n_tiles;
    int grid = sm_count() * per_sm;
    if (grid > total)
        grid = total;
    if (tuning().debug)
        fprintf(stderr, "conv_umma<%d,%d,%d>: per_sm %d grid %d items %d (whole tiles %d, split %d) smem %d\n",
                BN, GEOM, (int)SPLITK, per_sm, grid, total, SPLITK ? p.full_tiles : total,
                SPLITK ? p.split : 1, SmemLayout<BN, GEOM>::kDynamic);
    launch_pdl(conv_umma_kernel<BN, GEOM, SPLITK>, dim3(grid), dim3(kThreads),
               (size_t)SmemLayout<BN, GEOM>::kDynamic, st, ma, mb, p);
    return check_launch("conv_umma");
}

// ------------------------------------------------------------------------------------------
// split-K for the last, partly filled wave of 128 x 256 tiles
// ------------------------------------------------------------------------------------------
// 196 tiles on 148 SMs take two waves with the second a third full. The tiles of that last
// wave can be cut along K into `split` parts, each a work item of its own, so that the wave
// takes 1/split of a tile's MMA time when the parts fit the SMs. Parts leave their int32
// accumulators in scratch slabs; the last part of a tile to finish sums them and runs the
// usual epilogue (integer sums: the result does not depend on the order).
//
// OFF unless MB200_CONV_SPLITK=2..4 asks for it: bit-exact, but measured SLOWER on the
// ResNet-18 layers at batch 256 (512->512 7x7: 30.5 -> 32.6 us; 256->256 14x14: 26.7 ->
// 41.4 us). A part of 6-12 pipeline steps is 2-5 us of MMAs, while its epilogue writes a
// 128 KB slab (four times the int8 tile) and the finisher reads `split` slabs back from L2
// with eight 16-byte loads in flight per thread: about 64 KB in flight per SM, some 6 us for
// 384 KB, all of it after the last MMA of the kernel with nothing left to overlap it.
constexpr int kMaxSplitItems = 2 * 148;
constexpr size_t kSlabBytes = (size_t)kBM * 256 * 4;
constexpr size_t kCounterBytes = 4096;  // one word per split tile (fewer than 148)
constexpr size_t kSplitScratchBytes = kCounterBytes + kMaxSplitItems * kSlabBytes;

struct SplitPlan {
    int full_tiles, split, k_per_part, total_items;
};

SplitPlan plan_split_k(int tiles, int k_iters, int ctas) {
    SplitPlan sp{tiles, 1, k_iters, tiles};
    const int forced = tuning().conv_splitk;  // 2..4: that split wherever it fits
    if (forced < 2 || ctas <= 0)
        return sp;
    const int rem = tiles % ctas;
    if (rem == 0)
        return sp;
    int best = 1;
    for (int s = 2; s <= 4; ++s) {
        const int per_part = (k_iters + s - 1) / s;
        if (k_iters / s < 4 || (s - 1) * per_part >= k_iters ||  // no short or empty part
            rem * s > kMaxSplitItems || rem > (int)(kCounterBytes / 4))
            continue;
        if (forced == s)
            best = s;
    }
    if (best > 1) {
        sp.full_tiles = tiles - rem;
        sp.split = best;
        sp.k_per_part = (k_iters + best - 1) / best;
        sp.total_items = sp.full_tiles + rem * best;
    }
    return sp;
}

// Scratch for the slabs: one buffer per (device, stream), so that launches on different
// streams cannot meet in it; allocated at first use, never while the stream is capturing
// (the caller then runs unsplit). The counters at its start are zeroed once: every launch
// leaves them at zero.
void* split_scratch(cudaStream_t st) {
    static std::mutex mu;
    static std::map<std::pair<int, cudaStream_t>, void*> pool;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess)
        return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    auto it = pool.find(std::make_pair(dev, st));
    if (it != pool.end())
        return it->second;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
        cudaGetLastError();
        return nullptr;
    }
    void* ptr = nullptr;
    if (cudaMalloc(&ptr, kSplitScratchBytes) != cudaSuccess ||
        cudaMemset(ptr, 0, kCounterBytes) != cudaSuccess) {
        cudaGetLastError();
        if (ptr)
            cudaFree(ptr);
        ptr = nullptr;
    }
    pool[std::make_pair(dev, st)] = ptr;
    return ptr;
}

}  // namespace

// 1x1 filter, stride 1, no padding, NHWC: the convolution is a matrix product over the
// activation as it lies in memory
static bool conv_is_plain_matrix(const ConvArgs& a) {
    return a.kh == 1 && a.kw == 1 && a.sh == 1 && a.sw == 1 && a.ph == 0 && a.pw == 0 &&
           !a.src_is_nchw;
}

bool conv_umma_supported(
        const ConvArgs& a, const int8_t* src, const int8_t* flt, const int8_t* dst) {
    if (a.groups != 1 || a.src_is_nchw)
        return false;
    if (a.ic % kBK != 0)
        return false;
    if (a.kh * a.kw > 49 || a.dh != 1 || a.dw != 1)
        return false;
    // im2col bounding-box corners and tap offsets are 8-bit fields for a 4-D map
    if (a.ph > 64 || a.pw > 64 || a.kh > 64 || a.kw > 64 || a.sh > 8 || a.sw > 8)
        return false;
    // im2col maps are built over at least 128 KiB (descriptor_images); a pointwise
    // convolution uses a tiled map over the plain matrix and has no such limit
    if (!conv_is_plain_matrix(a) && descriptor_images(a, src) == 0)
        return false;
    if (((uintptr_t)src | (uintptr_t)flt | (uintptr_t)dst) & 15)
        return false;
    return true;
}

// geom: 0 = WIDE (src NHWC with ic % 64 == 0, filter [OC][KH][KW][IC]);
//       1 = TAP16 (src NHWC with exactly 16 channels, stride 1, filter [OC][taps][16] with the
//           tap count a multiple of 4; `a` then describes that transformed convolution, with
//           a.ph/a.pw the LOW padding and a.oh/a.ow the output extent)
int launch_conv_umma_geom(
        const ConvArgs& a, int geom_in, const int8_t* src, const int8_t* flt, const int32_t* bias,
        const float* flt_scales, int8_t* dst, cudaStream_t st) {
    int geom = geom_in;
    const DriverApi& api = driver_api();
    if (!api.ok)
        return set_error(ST_RUNTIME, "cuTensorMapEncode* entry points not found in the driver");
    const int taps = a.kh * a.kw;
    if (geom == GEOM_TAP16 && (a.ic != 16 || taps % 4 != 0 || a.sh != 1 || a.sw != 1))
        return set_error(ST_INVALID_LAYOUT, "TAP16 geometry needs 16 channels and 4k taps");
    if (((uintptr_t)bias & 15) || ((uintptr_t)flt_scales & 15))
        return set_error(ST_INVALID_LAYOUT, "bias and channel scales must be 16-byte aligned");

    // 128-channel rows whenever the channel count allows: fewer, larger TMA requests
    if (geom == GEOM_WIDE && a.ic % 128 == 0 && tuning().wide128)
        geom = GEOM_WIDE128;
    // MB200_CONV_PAIR=1: one 256 x 256 tile per pair of SMs (conv_pair.cu) wherever it applies.
    // Off by default: both kernels are bound by shared-memory bandwidth (operand reads of
    // the MMAs plus the TMA writes), and on the ResNet layers the pair measured no faster
    // than the 128 x 256 tile of a single SM.
    if (geom == GEOM_WIDE128 && conv_pair_supported(a, src, flt, dst)) {
        if (tuning().conv_pair != 0)
            return launch_conv_pair(a, src, flt, bias, flt_scales, dst, st);
    }
    const int chans = geom == GEOM_WIDE128 ? 128 : geom == GEOM_WIDE ? kBK : 16;
    int bn = a.oc <= 64 ? 64 : 128;
    {
        // 256 output channels per tile when the K loop is long enough to hide the epilogue
        // of a single CTA per SM and there are tiles for every SM
        const long long k_bytes = (long long)taps * a.ic;
        const long long tiles256 = (long long)((a.m + kBM - 1) / kBM) * ((a.oc + 255) / 256);
        const int force = tuning().conv_bn;
        if (geom == GEOM_WIDE128 && a.oc > 128 && k_bytes >= 1024 && tiles256 >= sm_count())
            bn = 256;
        if (force == 256 && geom == GEOM_WIDE128 && a.oc > 128)
            bn = 256;
        if (force == 128 && a.oc > 64)
            bn = 128;
        // A short K loop leaves the kernel to its epilogue warps: 64-column tiles hold half
        // the TMEM, so three CTAs (24 epilogue warps) fit an SM instead of two
        if (force == 64 || (force == 0 && k_bytes <= 256 && bn == 128))
            bn = 64;
    }
    const CUtensorMapSwizzle swz = geom == GEOM_WIDE128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                   : geom == GEOM_WIDE  ? CU_TENSOR_MAP_SWIZZLE_64B
                                                        : CU_TENSOR_MAP_SWIZZLE_NONE;
    CUtensorMap map_a, map_b;
    const bool a_tiled = geom != GEOM_TAP16 && conv_is_plain_matrix(a);
    if (a_tiled) {
        // a pointwise convolution reads the activation as the matrix [N*H*W][IC]: a tiled
        // map, 128 rows per box (rows past the end are filled with zeros)
        cuuint64_t dims[2] = {(cuuint64_t)a.ic, (cuuint64_t)a.m};
        cuuint64_t strides[1] = {(cuuint64_t)a.ic};
        cuuint32_t box[2] = {(cuuint32_t)chans, (cuuint32_t)kBM};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = api.tiled(
                &map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)src, dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return set_error(ST_RUNTIME, "cuTensorMapEncodeTiled(activation) failed: %d", (int)r);
    } else {
        // (a small activation is described with the images of readable memory behind it)
        const int images = descriptor_images(a, src);
        if (images == 0)
            return set_error(ST_INVALID_LAYOUT, "activation below 128 KiB outside a registered range");
        cuuint64_t dims[4] = {(cuuint64_t)a.ic, (cuuint64_t)a.iw, (cuuint64_t)a.ih,
                              (cuuint64_t)images};
        cuuint64_t strides[3] = {(cuuint64_t)a.ic, (cuuint64_t)a.iw * a.ic,
                                 (cuuint64_t)a.ih * a.iw * a.ic};
        // bounding box of the first-tap positions: from -pad to the last output's position
        int lower[2] = {-a.pw, -a.ph};
        int upper[2] = {(a.ow - 1) * a.sw - a.pw - (a.iw - 1), (a.oh - 1) * a.sh - a.ph - (a.ih - 1)};
        cuuint32_t estr[4] = {1, (cuuint32_t)a.sw, (cuuint32_t)a.sh, 1};
        CUresult r = api.im2col(
                &map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)src, dims, strides, lower, upper,
                chans, kBM, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return set_error(ST_RUNTIME, "cuTensorMapEncodeIm2col failed: %d", (int)r);
    }
    {
        const cuuint64_t k_total = (cuuint64_t)taps * a.ic;
        cuuint64_t dims[2] = {k_total, (cuuint64_t)a.oc};
        cuuint64_t strides[1] = {k_total};
        cuuint32_t box[2] = {(cuuint32_t)chans, (cuuint32_t)bn};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = api.tiled(
                &map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)flt, dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return set_error(ST_RUNTIME, "cuTensorMapEncodeTiled failed: %d", (int)r);
    }

    UmmaConvParams p;
    p.m_total = a.m;
    p.oc = a.oc;
    p.oh = a.oh;
    p.ow = a.ow;
    p.cblocks = geom == GEOM_TAP16 ? 1 : a.ic / chans;
    p.taps_w = a.kw;
    p.k_iters = geom == GEOM_TAP16 ? taps / 4 : taps * p.cblocks;
    p.sh = a.sh;
    p.sw = a.sw;
    p.base_h = -a.ph;
    p.base_w = -a.pw;
    p.dh = a.dh;
    p.dw = a.dw;
    p.m_tiles = (a.m + kBM - 1) / kBM;
    p.n_tiles = (a.oc + bn - 1) / bn;
    p.a_tiled = a_tiled ? 1 : 0;
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
    if (tuning().debug)
        fprintf(stderr, "%s: scales %g %g %g act %d z_mode %d verified requant: %d ops, %g + %.9g, short residual %g %g\n", "conv_umma",
                a.s_src, a.s_flt, a.s_dst, a.act, p.ep.z_mode, p.ep.fast_ops, p.ep.fast_mul, p.ep.fast_add,
                p.ep.z_fast_a,
                p.ep.z_fast_b);
    p.ep.acc_out = a.acc_out;
    p.dst = dst;
    p.status = device_status_word(st);
    p.wait_cycles = a.test_wait_cycles > 0 ? a.test_wait_cycles : kWaitCycles;
    p.skip_step = a.test_wait_cycles > 0 ? a.test_skip_step : -1;
    if (!p.status)
        return ST_MALLOC;
    p.full_tiles = p.total_items = p.m_tiles * p.n_tiles;
    p.split = 1;
    p.k_per_part = p.k_iters;
    p.slabs = nullptr;
    p.overlap = tuning().overlap_loads;
    p.counters = nullptr;
    if (geom == GEOM_WIDE128) {
        if (bn == 256) {
            const SplitPlan sp = plan_split_k(p.m_tiles * p.n_tiles, p.k_iters, sm_count());
            void* scratch = sp.split > 1 ? split_scratch(st) : nullptr;
            if (scratch) {
                p.full_tiles = sp.full_tiles;
                p.split = sp.split;
                p.k_per_part = sp.k_per_part;
                p.total_items = sp.total_items;
                p.counters = (unsigned*)scratch;
                p.slabs = (int4*)((uint8_t*)scratch + kCounterBytes);
                return launch_kernel<256, GEOM_WIDE128, true>(map_a, map_b, p, st);
            }
            return launch_kernel<256, GEOM_WIDE128>(map_a, map_b, p, st);
        }
        return bn == 64 ? launch_kernel<64, GEOM_WIDE128>(map_a, map_b, p, st)
                        : launch_kernel<128, GEOM_WIDE128>(map_a, map_b, p, st);
    }
    if (geom == GEOM_WIDE)
        return bn == 64 ? launch_kernel<64, GEOM_WIDE>(map_a, map_b, p, st)
                        : launch_kernel<128, GEOM_WIDE>(map_a, map_b, p, st);
    return bn == 64 ? launch_kernel<64, GEOM_TAP16>(map_a, map_b, p, st)
                    : launch_kernel<128, GEOM_TAP16>(map_a, map_b, p, st);
}

int launch_conv_umma(
        const ConvArgs& a, const int8_t* src, const int8_t* flt, const int32_t* bias,
        const float* flt_scales, int8_t* dst, cudaStream_t st) {
    return launch_conv_umma_geom(a, GEOM_WIDE, src, flt, bias, flt_scales, dst, st);
}

}  // namespace mb200
