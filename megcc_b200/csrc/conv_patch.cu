// qint8 ConvBias, stride 1, on the tensor cores with halo-patch input tiles and a filter that
// stays in shared memory.
//
// conv_umma.cu fetches the input once per filter tap (TMA im2col); for a 3x3 filter every
// pixel is requested nine times and the filter tile again for every output tile, and the
// request rate of the TMA unit becomes the limit. Here an output tile is a 16 (rows) x 8
// (columns) patch of one image, and its whole input neighbourhood, (16+KH-1) x (8+KW-1)
// pixels of all input channels, is brought in ONCE, by one TMA request, as planes of
// 16-channel chunks:
//
//     A stage  = [chunk = C/16][patch row][patch column][16 bytes]
//
// In the plain (unswizzled) K-major operand layout a core matrix is 8 rows x 16 bytes, rows
// 16 bytes apart: 8 horizontally adjacent pixels of one chunk plane are exactly that, and
// the next output row is PW*16 bytes further (the stride between 8-row groups). The operand
// of tap (fy, fx) is therefore the same planes addressed from pixel (fy, fx): every tap is
// a shifted view, nothing is copied or fetched again. (Core matrices that do not start on a
// 128-byte boundary cost the MMA nothing: a variant with one aligned copy per horizontal
// offset issued its MMAs at the same rate.) The CTA's filter slice [BN][KH*KW*C] is loaded
// once and stays resident; persistent CTAs walk the patch list.
//
// Accumulators: int32 in TMEM, two buffers; epilogue identical in arithmetic to conv_umma.cu
// (reference order of compiler/lib/KernelGen/BareMetal/Activation.cpp:105-113).
//
// POOL = 1 folds the MAX pooling 3x3 / stride 2 / pad 1 that follows the ConvBias into the
// epilogue (a ResNet stem). Requantisation with positive scales and IDENTITY / RELU is a
// non-decreasing function of the int32 accumulator, and the bias is one constant per channel,
// so max over a window of requantised values == requantised max of the accumulators, bit for
// bit: the window maximum is taken on the int32 accumulators (staged through shared memory)
// and only one value in four is requantised and stored; the full-resolution tensor never
// exists. A 16 x 8 patch of ConvBias outputs whose origin is the odd position (2P-1, 2Q-1)
// holds every window of a 7 x 3 block of pooled outputs, so patches are laid 14 x 6 apart
// and overlap by their last two rows / columns (0.66 of the MMA rows are distinct outputs).
#include <stdio.h>
#include <stdlib.h>

#include "conv_epilogue.cuh"
#include "internal.h"
#include "pdl.h"
#include "tuning.h"
#include "umma_ptx.cuh"

namespace mb200 {

using namespace umma;

namespace {

constexpr int kTH = 16, kTW = 8;  // output patch; kTW = 8 makes a patch row one core matrix
// Epilogue warps per CTA (EW): 8 (two per TMEM lane quarter) when several CTAs share an SM,
// 16 when the resident filter slice leaves room for one CTA only: that CTA then has the SM's
// registers and issue slots to itself, and a single CTA's eight warps cannot keep up with
// its own MMAs.
constexpr int kMaxStages = 3;

// pooled outputs per patch and the distance between patch origins (POOL form)
constexpr int kPoolRows = 7, kPoolCols = 3;
constexpr int kPoolBufBytes = 128 * 64 * 4;  // int32 accumulators of one 128 x 64 tile

struct PatchParams {
    int n, oh, ow, oc;
    int poh, pow;    // POOL form: extent of the pooled output
    int chunks;      // C / 16
    int kh, kw, ph, pw;
    int pph, ppw;    // input patch extent: kTH + kh - 1, kTW + kw - 1
    int tiles_y, tiles_x, m_tiles, n_tiles;
    int stages;
    int a_stage_bytes, a_tx_bytes, b_bytes;
    int plane_stride;  // one chunk plane: pph x ppw pixels of 16 bytes
    int b_single_load;  // the filter map is the 3-D view (one load) rather than 2-D blocks
    int a_flat16;       // 16 input channels: the activation map is {W * 16 bytes, H, N}
    int mma_per_tap;  // k-steps per tap (C/32), or 0 when C == 16 (two taps per k-step)
    int a_lbo;        // distance between the two 16-byte K halves of one A operand
    // Depthwise form (64-channel rows kernel only): the raw filter [C][3][3]. Each CTA then
    // convolves input channels n0 .. n0+63 with the block-diagonal operand it builds itself.
    int overlap;  // 1: chunks of the verified short forms load their accumulators in two halves
    const int8_t* dw_flt;
    // 1: the depthwise tensor has 32 channels and is seen as pixel PAIRS of 64 bytes
    // ([N][H][W/2][2][32]); column 32 h + c of a row is channel c of the pair's pixel h
    int dw_pairs;
    EpilogueParams ep;
    int8_t* dst;
    int* status;
};

// Position of a CTA's current patch (image, patch row, patch column) and the step to its
// next one, kept as three counters with carries: one division at the start, none per tile.
// (With 64 output channels an epilogue warp does one 32-column chunk per tile, so whatever
// the tile decode costs is paid per chunk.)
struct PatchWalker {
    int img, ty, tx;
    int s_img, s_ty, s_tx;
    int tiles_y, tiles_x;
    __device__ __forceinline__ PatchWalker(int first, int step, int ty_n, int tx_n)
            : tiles_y(ty_n), tiles_x(tx_n) {
        const int per_image = ty_n * tx_n;
        img = first / per_image;
        int r = first - img * per_image;
        ty = r / tx_n;
        tx = r - ty * tx_n;
        s_img = step / per_image;
        r = step - s_img * per_image;
        s_ty = r / tx_n;
        s_tx = r - s_ty * tx_n;
    }
    __device__ __forceinline__ void next() {
        tx += s_tx;
        if (tx >= tiles_x) {
            tx -= tiles_x;
            ++ty;
        }
        ty += s_ty;
        if (ty >= tiles_y) {
            ty -= tiles_y;
            ++img;
        }
        img += s_img;
    }
};

// One tile's MMAs. The issuing thread runs alone in its warp and every instruction of its
// loop costs it several cycles, so the hot filter shapes get their own instantiation
// (KH > 0) where every operand offset is a compile-time constant: two adds per MMA. Looking
// the offsets up in a shared-memory table measured slower than the MMAs themselves.
template <int BN, int KH, int KW, int CHUNKS>
__device__ __forceinline__ void issue_tile_mmas(
        const PatchParams& p, uint64_t a0, uint64_t b0, uint32_t tmem_d) {
    constexpr uint32_t idesc = umma_idesc_s8(128, BN);
    // all offsets in descriptor address units (16 bytes = one pixel of one chunk plane)
    if constexpr (KH > 0) {
        constexpr uint32_t ppw = kTW + KW - 1;
        constexpr uint32_t plane16 = (kTH + KH - 1) * ppw;
        if constexpr (CHUNKS == 1) {
            // 16 channels: taps (fx, fx+1) are the two K halves; the second half is the
            // same plane one pixel to the right
#pragma unroll
            for (int fy = 0; fy < KH; ++fy) {
#pragma unroll
                for (int fx = 0; fx < KW; fx += 2) {
                    const uint64_t ad = a0 + (fy * ppw + fx), bd = b0 + (uint32_t)((fy * KW + fx) * BN);
                    if ((fy | fx) == 0)
                        umma_s8_c<false>(tmem_d, ad, bd, idesc);
                    else
                        umma_s8_c<true>(tmem_d, ad, bd, idesc);
                }
            }
        } else {
#pragma unroll
            for (int fy = 0; fy < KH; ++fy) {
#pragma unroll
                for (int fx = 0; fx < KW; ++fx) {
#pragma unroll
                    for (int j = 0; j < CHUNKS / 2; ++j) {
                        // chunks 2j, 2j+1 are the two 16-byte K halves of this step
                        const uint64_t ad = a0 + (fy * ppw + fx + 2 * j * plane16);
                        const uint64_t bd = b0 + (uint32_t)(((fy * KW + fx) * CHUNKS + 2 * j) * BN);
                        if ((fy | fx | j) == 0)
                            umma_s8_c<false>(tmem_d, ad, bd, idesc);
                        else
                            umma_s8_c<true>(tmem_d, ad, bd, idesc);
                    }
                }
            }
        }
    } else {
        const uint32_t plane16 = (uint32_t)p.plane_stride >> 4;
        uint32_t acc = 0;
        uint64_t b_desc = b0;
        if (p.mma_per_tap > 0) {
            for (int fy = 0; fy < p.kh; ++fy) {
                uint64_t a_tap = a0 + (uint32_t)(fy * p.ppw);
                for (int fx = 0; fx < p.kw; ++fx, ++a_tap) {
                    uint64_t a_desc = a_tap;
                    for (int j = 0; j < p.mma_per_tap; ++j, a_desc += 2 * plane16, b_desc += 2 * BN) {
                        umma_s8(tmem_d, a_desc, b_desc, idesc, acc);
                        acc = 1;
                    }
                }
            }
        } else {
            for (int fy = 0; fy < p.kh; ++fy) {
                uint64_t a_desc = a0 + (uint32_t)(fy * p.ppw);
                for (int fx = 0; fx < p.kw; fx += 2, a_desc += 2, b_desc += 2 * BN) {
                    umma_s8(tmem_d, a_desc, b_desc, idesc, acc);
                    acc = 1;
                }
            }
        }
    }
}

// The row form (ROWS = 1; 64 input channels): the patch is stored as [patch row][16 columns]
// [64 bytes] with the 64-byte swizzle, one TMA request whose rows are a pixel's 64 channels.
// The plain form above needs C/16 rows of 16 bytes per pixel, and the TMA unit's cost is per
// row: 720 rows per tile against 288 here. A patch row is padded to 16 columns so that the
// 8-row groups of a tap lie a multiple of the swizzle pattern (512 bytes) apart; the
// swizzle is a function of the shared-memory address, so a tap's shifted start needs
// nothing else. `a0` / `b0` are 64-byte-swizzle descriptors of the stage / filter base.
constexpr int kRowCols = 16;
template <int BN, int KH, int KW>
__device__ __forceinline__ void issue_tile_mmas_rows64(uint64_t a0, uint64_t b0, uint32_t tmem_d) {
    constexpr uint32_t idesc = umma_idesc_s8(128, BN);
    constexpr uint32_t pix16 = 64 / 16;  // one pixel in descriptor address units
#pragma unroll
    for (int fy = 0; fy < KH; ++fy) {
#pragma unroll
        for (int fx = 0; fx < KW; ++fx) {
#pragma unroll
            for (int k = 0; k < 2; ++k) {  // two K steps of 32 bytes inside the 64-byte row
                const uint64_t ad = a0 + (uint32_t)((fy * kRowCols + fx) * pix16 + 2 * k);
                const uint64_t bd = b0 + (uint32_t)((fy * KW + fx) * BN * pix16 + 2 * k);
                if ((fy | fx | k) == 0)
                    umma_s8_c<false>(tmem_d, ad, bd, idesc);
                else
                    umma_s8_c<true>(tmem_d, ad, bd, idesc);
            }
        }
    }
}

template <int BN, int KH, int KW, int CHUNKS, int EW, int ROWS = 0, int POOL = 0>
__global__ void __launch_bounds__(64 + 32 * EW, EW == 16 ? 1 : 2) conv_patch_kernel(
        const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
        const PatchParams p) {
    static_assert(POOL == 0 || (BN == 64 && EW == 8 && ROWS == 0), "pooled form: 64 channels");
    constexpr int kEpilogueWarps = EW;
    // distance between patch origins and the origin's offset (see the POOL note above)
    constexpr int kStepY = POOL ? 2 * kPoolRows : kTH, kStepX = POOL ? 2 * kPoolCols : kTW;
    constexpr int kOrigin = POOL ? -1 : 0;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_b = smem;
    uint8_t* smem_a = smem + p.b_bytes;
    uint64_t* bars = (uint64_t*)(smem_a + p.stages * p.a_stage_bytes);
    uint64_t* a_full = bars;                    // [kMaxStages]
    uint64_t* a_empty = a_full + kMaxStages;    // [kMaxStages]
    uint64_t* acc_full = a_empty + kMaxStages;  // [2]
    uint64_t* acc_empty = acc_full + 2;         // [2]
    uint64_t* b_full = acc_empty + 2;
    uint64_t* drain_bar = b_full + 1;
    uint32_t* tmem_slot = (uint32_t*)(drain_bar + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    // POOL: the tile's int32 accumulators, [pixel][16 groups of 4 channels], the group index
    // XORed with the pixel's column so that neither the row-wise writes nor the window reads
    // collide on banks
    uint8_t* pool_buf = (uint8_t*)(((uintptr_t)(abort_flag + 1) + 127) & ~(uintptr_t)127);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // each CTA owns one slice of output channels and walks the patches with a fixed stride
    const int tile_n = blockIdx.x % p.n_tiles;
    const int m_first = blockIdx.x / p.n_tiles;
    const int m_step = gridDim.x / p.n_tiles;
    const int n0 = tile_n * BN;
    const int plane = p.plane_stride;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(&a_full[s], 1);
            mbar_init(&a_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 32 * kEpilogueWarps);  // every epilogue thread arrives
        }
        mbar_init(b_full, 1);
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if constexpr (ROWS != 0) {
        if (p.dw_flt) {
            // Depthwise 3x3 as a dense 64 -> 64 convolution of this CTA's channel slice with
            // a block-diagonal filter: tap t is the [64 oc][64 ic] tile whose only non-zero
            // bytes are w[n0 + c][t] at (c, c). Written here in the layout the TMA would have
            // produced (rows of 64 bytes, 64-byte swizzle: 16-byte unit u of row r sits at
            // unit u ^ ((r >> 1) & 3)), then handed to the tensor core's (async) proxy.
            uint4* b16 = reinterpret_cast<uint4*>(smem_b);
            for (int i = threadIdx.x; i < 9 * BN * 4; i += blockDim.x)
                b16[i] = make_uint4(0, 0, 0, 0);
            __syncthreads();
            for (int i = threadIdx.x; i < 9 * BN; i += blockDim.x) {
                const int t = i / BN, c = i - t * BN;  // tap, output column (tile row)
                uint8_t* row = smem_b + t * (BN * 64) + c * 64;
                const int swz = (c >> 1) & 3;
                if (!p.dw_pairs) {
                    row[(((c >> 4) ^ swz) << 4) + (c & 15)] =
                            (uint8_t)p.dw_flt[(size_t)(n0 + c) * 9 + t];
                } else {
                    // Pixel pairs: output pixel ho of pair x sees input pixel hi of pair
                    // x + fx - 1 through filter column dx = 2 (fx - 1) + hi - ho + 1.
                    const int fy = t / 3, fx = t - fy * 3, ho = c >> 5, ch = c & 31;
#pragma unroll
                    for (int hi = 0; hi < 2; ++hi) {
                        const int dx = 2 * (fx - 1) + hi - ho + 1;
                        if (dx >= 0 && dx <= 2) {
                            const int k = hi * 32 + ch;  // input column
                            row[(((k >> 4) ^ swz) << 4) + (k & 15)] =
                                    (uint8_t)p.dw_flt[ch * 9 + fy * 3 + dx];
                        }
                    }
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
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
    pdl_release();  // the next kernel may be scheduled onto SMs this one leaves

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            // the filter slice, once: one [BN][16-byte] block per 16 bytes of K (weights: they
            // do not depend on the kernel before this one, so they are fetched before the wait)
            const int kchunks = p.kh * p.kw * p.chunks;
            if (ROWS && p.dw_flt) {
                mbar_arrive(b_full);  // the operand was built in place before the roles split
            } else if (ROWS) {
                mbar_expect_tx(b_full, (uint32_t)p.b_bytes);
                // one swizzled [BN][64-byte] tile per filter tap
                for (int t = 0; t < p.kh * p.kw; ++t)
                    tma_load_2d(smem_b + t * (BN * 64), &map_b, b_full, t * 64, n0);
            } else if (p.b_single_load) {
                // 3-D view {16 bytes, rows, K/16}: one request lays down every block
                mbar_expect_tx(b_full, (uint32_t)p.b_bytes);
                tma_load_3d(smem_b, &map_b, b_full, 0, n0, 0);
            } else {
                mbar_expect_tx(b_full, (uint32_t)p.b_bytes);
                for (int kc = 0; kc < kchunks; ++kc)
                    tma_load_2d(smem_b + kc * (BN * 16), &map_b, b_full, kc * 16, n0);
            }
            pdl_wait();  // activations: only once the previous kernel has completed
            int s = 0;
            uint32_t phase = 0;
            PatchWalker at(m_first, m_step, p.tiles_y, p.tiles_x);
            for (int mt = m_first; mt < p.m_tiles; mt += m_step, at.next()) {
                if (!mbar_wait(&a_empty[s], phase ^ 1u, abort_flag)) {
                    if (!*abort_flag) {
                        *abort_flag = 1;
                        atomicExch(p.status, ERR_PRODUCER_WAIT);
                    }
                    break;
                }
                const int img = at.img;
                const int x0 = at.tx * kStepX + kOrigin - p.pw, y0 = at.ty * kStepY + kOrigin - p.ph;
                mbar_expect_tx(&a_full[s], (uint32_t)p.a_tx_bytes);
                if (ROWS) {
                    // one request: box {64 B, 16 columns, patch rows, 1 image} (depthwise
                    // form: this CTA's 64 input channels)
                    tma_load_4d(smem_a + s * p.a_stage_bytes, &map_a, &a_full[s], p.dw_flt ? n0 : 0,
                                x0, y0, img);
                } else if (p.a_flat16) {
                    // 16 channels: a patch row is contiguous in memory, one box row of
                    // (patch columns x 16) bytes instead of one 16-byte row per pixel (the
                    // TMA unit's cost is per row)
                    tma_load_3d(smem_a + s * p.a_stage_bytes, &map_a, &a_full[s], x0 * 16, y0, img);
                } else {
                    // one request: box {16 B, patch columns, patch rows, 1 image, all chunks}
                    tma_load_5d(smem_a + s * p.a_stage_bytes, &map_a, &a_full[s], 0, x0, y0, img, 0);
                }
                if (++s == p.stages) {
                    s = 0;
                    phase ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            bool ok = mbar_wait(b_full, 0, abort_flag);
            if (!ok && !*abort_flag) {
                *abort_flag = 1;
                atomicExch(p.status, ERR_MMA_WAIT);
            }
            const uint32_t sbo_a = (uint32_t)p.ppw * 16;  // the next patch row
            const uint64_t b0 = ROWS ? umma_smem_desc(smem_u32(smem_b), 16, 512, 4)
                                     : umma_smem_desc(smem_u32(smem_b), BN * 16, 128, 0);
            int local = 0, s = 0;
            uint32_t phase = 0;
            for (int mt = m_first; mt < p.m_tiles && ok; mt += m_step, ++local) {
                const int buf = local & 1;
                const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
                if (!mbar_wait(&acc_empty[buf], acc_phase ^ 1u, abort_flag)) {
                    if (!*abort_flag) {
                        *abort_flag = 1;
                        atomicExch(p.status, ERR_MMA_ACC_WAIT);
                    }
                    break;
                }
                if (!mbar_wait(&a_full[s], phase, abort_flag)) {
                    if (!*abort_flag) {
                        *abort_flag = 1;
                        atomicExch(p.status, ERR_MMA_WAIT);
                    }
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_u32(smem_a + s * p.a_stage_bytes);
                const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
                if constexpr (ROWS != 0) {
                    // 8-row groups (patch rows) are 16 pixels x 64 bytes apart
                    const uint64_t a0 = umma_smem_desc(a_addr, 16, kRowCols * 64, 4);
                    issue_tile_mmas_rows64<BN, KH, KW>(a0, b0, tmem_d);
                } else {
                    const uint64_t a0 = umma_smem_desc(a_addr, (uint32_t)p.a_lbo, sbo_a, 0);
                    issue_tile_mmas<BN, KH, KW, CHUNKS>(p, a0, b0, tmem_d);
                }
                umma_commit(&a_empty[s]);
                umma_commit(&acc_full[buf]);
                if (++s == p.stages) {
                    s = 0;
                    phase ^= 1u;
                }
            }
        }
    } else {
        // ---------------- epilogue ----------------
        pdl_wait();  // before the first read of z and the first store over memory in use
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const int py = row >> 3, px = row & 7;
        int local = 0;
        bool ok = true;
        // POOL: this thread's channel group (4 channels) and first pooled pixel of a patch;
        // its bias and filter scales do not change from patch to patch
        const int pool_g = (int)(threadIdx.x - 64) & 15, pool_pj = (int)(threadIdx.x - 64) >> 4;
        const int pool_ch = n0 + pool_g * 4;
        int4 pool_bias = make_int4(0, 0, 0, 0);
        float4 pool_scales = make_float4(0.f, 0.f, 0.f, 0.f);
        if (POOL != 0 && pool_ch < p.oc) {
            if (p.ep.bias)
                pool_bias = __ldg(reinterpret_cast<const int4*>(p.ep.bias + pool_ch));
            if (p.ep.flt_scales)
                pool_scales = __ldg(reinterpret_cast<const float4*>(p.ep.flt_scales + pool_ch));
        }
        const bool overlap_ok = POOL == 0 && p.overlap && epilogue_chunk_overlappable(p.ep, p.dst, 0);
        PatchWalker at(m_first, m_step, p.tiles_y, p.tiles_x);
        for (int mt = m_first; mt < p.m_tiles && ok; mt += m_step, ++local, at.next()) {
            const int buf = local & 1;
            const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
            ok = mbar_wait(&acc_full[buf], acc_phase, abort_flag);
            if (!ok && !*abort_flag) {
                *abort_flag = 1;
                atomicExch(p.status, ERR_EPILOGUE_WAIT);
            }
            if constexpr (POOL != 0) {
                // The epilogue warps meet at barriers below, so they must leave the loop
                // together: agree on the outcome of the (bounded) wait across all of them.
                // Arriving here also says that this thread is through with the staging
                // buffer of the previous tile.
                int all;
                asm volatile(
                        "{\n\t.reg .pred p, r;\n\tsetp.ne.u32 p, %1, 0;\n\t"
                        "bar.red.and.pred r, 1, %2, p;\n\tselp.u32 %0, 1, 0, r;\n\t}"
                        : "=r"(all)
                        : "r"((int)ok), "n"(32 * EW)
                        : "memory");
                ok = all != 0;
            } else {
                ok = __all_sync(0xffffffffu, ok);
            }
            if (!ok)
                break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if constexpr (POOL != 0) {
                // (1) this thread's pixel: 32 accumulators TMEM -> registers -> shared memory
                const int c = (warp - 2) >> 2;  // the warp's 32-column chunk
                {
                    uint32_t v[32];
                    tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN) +
                                      (uint32_t)(c * 32),
                              v);
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    mbar_arrive(&acc_empty[buf]);
                    // a position outside the ConvBias output (the rim of the first / last
                    // patches) must never win a window: the smallest int32 in its place.
                    // (Every window's centre is a real output, so that value never reaches
                    // the bias addition.)
                    const int oy = at.ty * kStepY + kOrigin + py, ox = at.tx * kStepX + kOrigin + px;
                    if ((unsigned)oy >= (unsigned)p.oh || (unsigned)ox >= (unsigned)p.ow) {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            v[j] = 0x80000000u;
                    }
                    uint8_t* mine = pool_buf + row * 256;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int g = c * 8 + (j ^ px);  // group c*8+j at slot (c*8+j) ^ px
                        *reinterpret_cast<uint4*>(mine + g * 16) =
                                make_uint4(v[j * 4], v[j * 4 + 1], v[j * 4 + 2], v[j * 4 + 3]);
                    }
                }
                asm volatile("bar.sync 1, %0;" ::"n"(32 * EW) : "memory");
                // (2) one pooled pixel x 4 channels per item, 21 x 16 items over the 256
                // threads: 16 consecutive lanes read the 16 groups of one pixel (every slot of
                // its 256 bytes once: no bank conflicts) and store its 64 bytes
#pragma unroll 1
                for (int pj = pool_pj; pj < kPoolRows * kPoolCols; pj += 16) {
                    const int pyj = pj / kPoolCols, pxj = pj - pyj * kPoolCols;
                    const int P = at.ty * kPoolRows + pyj, Q = at.tx * kPoolCols + pxj;
                    if (P >= p.poh || Q >= p.pow)
                        continue;
                    // the window: 3 x 3 pixels from (2 pyj, 2 pxj); a pixel's group sits at
                    // the slot XORed with the pixel's column
                    const uint8_t* win = pool_buf + (2 * pyj * 8 + 2 * pxj) * 256;
                    const uint8_t* col[3];
#pragma unroll
                    for (int wx = 0; wx < 3; ++wx)
                        col[wx] = win + wx * 256 + ((pool_g ^ (2 * pxj + wx)) << 4);
                    uint32_t m[4];
#pragma unroll
                    for (int wy = 0; wy < 3; ++wy) {
#pragma unroll
                        for (int wx = 0; wx < 3; ++wx) {
                            const uint4 t = *reinterpret_cast<const uint4*>(col[wx] + wy * 8 * 256);
                            if (wy == 0 && wx == 0) {
                                m[0] = t.x, m[1] = t.y, m[2] = t.z, m[3] = t.w;
                            } else {
                                m[0] = (uint32_t)max((int)m[0], (int)t.x);
                                m[1] = (uint32_t)max((int)m[1], (int)t.y);
                                m[2] = (uint32_t)max((int)m[2], (int)t.z);
                                m[3] = (uint32_t)max((int)m[3], (int)t.w);
                            }
                        }
                    }
                    const uint32_t pixel = ((uint32_t)at.img * p.poh + P) * p.pow + Q;
                    if (pool_ch < p.oc)
                        *reinterpret_cast<uint32_t*>(p.dst + (size_t)pixel * p.oc + pool_ch) =
                                epilogue_word(m, pool_bias, pool_scales, p.ep);
                }
                continue;  // (the next tile's agreement barrier frees the staging buffer)
            }
            const int oy = at.ty * kTH + py, ox = at.tx * kTW + px;
            const bool valid = oy < p.oh && ox < p.ow;
            // the pixel index fits 32 bits (the launcher checks); one wide multiply
            const uint32_t pixel = ((uint32_t)at.img * p.oh + oy) * p.ow + ox;
            const size_t px_off = (size_t)pixel * p.oc;
            if (p.ep.z_mode != 0) {
                // The residual operand is the one read of this epilogue that nothing
                // pipelines: ask for the bytes this thread will want one tile from now, so
                // that they wait in L2 instead of DRAM when the chunk below loads them.
                PatchWalker nx = at;
                nx.next();
                const int ny = nx.ty * kTH + py, nxx = nx.tx * kTW + px;
                if (mt + m_step < p.m_tiles && ny < p.oh && nxx < p.ow) {
                    const uint32_t npix = ((uint32_t)nx.img * p.oh + ny) * p.ow + nxx;
                    const int8_t* zn = p.ep.z + (size_t)npix * p.oc + n0 + ((warp - 2) >> 2) * 32;
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(zn));
                }
            }
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
            const int half = (warp - 2) >> 2;
            // each warp takes a run of adjacent chunks: its thread's bytes are contiguous
            constexpr int kChunksPerWarp = (BN / 32) / (kEpilogueWarps / 4);
            static_assert(kChunksPerWarp >= 1, "every epilogue warp must own a chunk: it is "
                                               "counted on the accumulator-drained barrier");
            // one 32-column chunk: registers <- TMEM, buffer released after the warp's last
            // load, requantisation, store
            auto do_chunk = [&](int c, bool last) {
                if (overlap_ok && n0 + c * 32 + 32 <= p.oc) {
                    // a verified short form: the chunk's second 16 columns are fetched while
                    // the first are requantised
                    const int ch0 = n0 + c * 32;
                    epilogue_chunk_overlapped(
                            taddr + (uint32_t)(c * 32), p.ep, p.dst, px_off + ch0,
                            (ROWS != 0 && p.dw_pairs) ? (ch0 & 31) : ch0, valid,
                            last ? &acc_empty[buf] : nullptr);
                    return;
                }
                uint32_t v[32];
                tmem_ld32(taddr + (uint32_t)(c * 32), v);
                if (last) {
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    mbar_arrive(&acc_empty[buf]);
                }
                const int ch0 = n0 + c * 32;
                if (valid && ch0 < p.oc)
                    // (pixel pairs: bias and channel scales are those of channel column % 32)
                    epilogue_store<32>(v, p.ep, p.dst, px_off + ch0,
                                       (ROWS != 0 && p.dw_pairs) ? (ch0 & 31) : ch0);
            };
            if constexpr (kChunksPerWarp == 1) {
                // Written as a strided loop of (at run time) one trip: with the chunk's code
                // inlined straight into the tile loop the compiler spills 2 KB per thread
                // per tile at 64 registers, and the 64-channel kernels run 5 % slower.
                constexpr int kChunkStep = kEpilogueWarps / 4;
#pragma unroll 1
                for (int c = half; c < BN / 32; c += kChunkStep)
                    do_chunk(c, c + kChunkStep >= BN / 32);
            } else {
#pragma unroll 1
                for (int c = half * kChunksPerWarp; c < (half + 1) * kChunksPerWarp; ++c)
                    do_chunk(c, c + 1 == (half + 1) * kChunksPerWarp);
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
                     "r"(2 * BN)
                     : "memory");
    }
}

struct PatchPlan {
    bool ok;
    int bn, stages, ctas_per_sm;
    int a_stage_bytes, b_bytes, smem_bytes, plane_stride;
    bool rows64;  // 64-channel 3x3: pixel rows of 64 bytes, 64-byte swizzle
};

// CTAs per SM to try first; MB200_PATCH_CTAS overrides (performance experiments)
int patch_first_ctas() {
    const int v = tuning().patch_ctas;
    return v >= 1 && v <= 3 ? v : 3;
}

PatchPlan plan_patch(const ConvArgs& a) {
    PatchPlan pl{};
    if (a.groups != 1 || a.src_is_nchw || a.sh != 1 || a.sw != 1 || a.dh != 1 || a.dw != 1)
        return pl;
    if (a.ic % 16 != 0 || a.ic > 128 || (a.ic != 16 && a.ic % 32 != 0))
        return pl;
    if (a.ic == 16 && a.kw % 2 != 0)
        return pl;
    if (a.kh > 8 || a.kw > 8 || a.ph > 8 || a.pw > 8)
        return pl;
    const int pph = kTH + a.kh - 1, ppw = kTW + a.kw - 1;
    if (pph > 256 || ppw > 256)
        return pl;
    pl.bn = (a.oc <= 64 || a.dw64) ? 64 : 128;
    if (a.pool && (pl.bn != 64 || a.oc % 16 != 0))
        return pl;
    pl.rows64 = a.ic == 64 && a.kh == 3 && a.kw == 3 && pl.bn == 64 &&
                (!tuning().patch_plain || a.dw64) && !a.pool;
    if (a.dw64 && (!pl.rows64 || a.oc % 64 != 0 || a.acc_out))
        return pl;
    pl.plane_stride = pph * ppw * 16;
    // a TMA destination in shared memory must be 128-byte aligned: pad the stage
    pl.a_stage_bytes = ((a.ic / 16) * pl.plane_stride + 127) / 128 * 128;
    if (pl.rows64)
        pl.a_stage_bytes = pph * kRowCols * 64;  // a multiple of 1024
    pl.b_bytes = pl.bn * a.kh * a.kw * a.ic;
    const int fixed = pl.b_bytes + (2 * kMaxStages + 6) * 8 + 64 + 1024 +
                      (a.pool ? kPoolBufBytes + 128 : 0);
    const int budget = 227 * 1024;
    // more CTAs per SM hide more latency; one stage is a whole tile, so two stages already
    // keep the loads a tile ahead
    const int min_stages = 2;
    for (int per_sm = patch_first_ctas(); per_sm >= 1; --per_sm) {
        const int avail = budget / per_sm - 1024 - fixed;
        int st = avail / pl.a_stage_bytes;
        if (st > kMaxStages)
            st = kMaxStages;
        if (st >= min_stages && 2 * pl.bn * per_sm <= 512) {
            pl.ok = true;
            pl.stages = st;
            pl.ctas_per_sm = per_sm;
            pl.smem_bytes = fixed + st * pl.a_stage_bytes;
            return pl;
        }
    }
    return pl;
}

template <int BN, int KH, int KW, int CHUNKS, int EW, int ROWS = 0, int POOL = 0>
int launch_patch(
        const CUtensorMap& ma, const CUtensorMap& mb, const PatchParams& p, int smem, int grid,
        cudaStream_t st) {
    constexpr int kThreads = 64 + 32 * EW;
    if (cudaFuncSetAttribute(
                conv_patch_kernel<BN, KH, KW, CHUNKS, EW, ROWS, POOL>,
                cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return check_launch("conv_patch smem attribute");
    // never more CTAs than are resident at once: a persistent CTA that starts late would
    // leave its share of the patches to the end
    const int per_sm = resident_ctas_per_sm(conv_patch_kernel<BN, KH, KW, CHUNKS, EW, ROWS, POOL>,
                                            kThreads, smem, 2 * BN);
    {
        int cap = sm_count() * per_sm / p.n_tiles * p.n_tiles;
        if (cap >= p.n_tiles && grid > cap)
            grid = cap;
    }
    if (tuning().debug)
        fprintf(stderr, "conv_patch<%d,%d,%d,%d,%d,%d,%d>: per_sm %d grid %d m_tiles %d n_tiles %d "
                "smem %d stages %d b_single_load %d\n", BN, KH, KW, CHUNKS, EW, ROWS, POOL, per_sm,
                grid, p.m_tiles, p.n_tiles, smem, p.stages, p.b_single_load);
    launch_pdl(conv_patch_kernel<BN, KH, KW, CHUNKS, EW, ROWS, POOL>, dim3(grid), dim3(kThreads),
               (size_t)smem, st, ma, mb, p);
    return check_launch("conv_patch");
}

}  // namespace

// Fraction of the MMA rows that land on real output pixels; the caller weighs it against
// the im2col kernel, which has no such loss.
float conv_patch_efficiency(const ConvArgs& a) {
    // A filter slice so large that one CTA has the SM to itself leaves a single thread to
    // issue every MMA of the SM, and with 128-column MMAs (64 cycles each) that thread, which
    // shares its scheduler with epilogue warps, is the limit: the im2col kernel with two CTAs
    // per SM measured faster. MB200_PATCH_ALONE=1 uses the patch kernel all the same.
    if (plan_patch(a).ctas_per_sm < 2) {
        if (!tuning().patch_alone)
            return 0.f;
    }
    const int ty = (a.oh + kTH - 1) / kTH, tx = (a.ow + kTW - 1) / kTW;
    return (float)(a.oh * a.ow) / (float)(ty * kTH * tx * kTW);
}

bool conv_patch_supported(
        const ConvArgs& a, const int8_t* src, const int8_t* flt, const int8_t* dst) {
    if (!plan_patch(a).ok)
        return false;
    if (descriptor_images(a, src) == 0)  // maps are built over at least 128 KiB
        return false;
    if ((size_t)a.n * a.oh * a.ow >= (1ull << 31))
        return false;
    if (((uintptr_t)src | (uintptr_t)flt | (uintptr_t)dst) & 15)
        return false;
    // the fused pooling commutes with the requantisation only where that is non-decreasing
    if (a.pool && (a.act == ACT_H_SWISH || a.z || a.acc_out || !(a.s_src > 0.f) ||
                   !(a.s_flt > 0.f) || !(a.s_dst > 0.f)))
        return false;
    return true;
}

// `a`: stride-1 dense convolution over an NHWC source; a.ph / a.pw are the LOW paddings and
// a.oh / a.ow the output extent (the upper padding is whatever those imply).
int launch_conv_patch(
        const ConvArgs& a, const int8_t* src, const int8_t* flt, const int32_t* bias,
        const float* flt_scales, int8_t* dst, cudaStream_t st) {
    const DriverApi& api = driver_api();
    if (!api.ok)
        return set_error(ST_RUNTIME, "cuTensorMapEncode* entry points not found in the driver");
    const PatchPlan pl = plan_patch(a);
    if (!pl.ok)
        return set_error(ST_NO_IMPLEMENT, "halo-patch ConvBias does not apply to this shape");
    if (((uintptr_t)bias & 15) || ((uintptr_t)flt_scales & 15))
        return set_error(ST_INVALID_LAYOUT, "bias and channel scales must be 16-byte aligned");

    const int pph = kTH + a.kh - 1, ppw = kTW + a.kw - 1;
    // (a small activation is described with the images of readable memory behind it)
    const int images = descriptor_images(a, src);
    if (images == 0)
        return set_error(ST_INVALID_LAYOUT, "activation below 128 KiB outside a registered range");
    CUtensorMap map_a, map_b;
    if (pl.rows64) {
        // (depthwise form: the tensor has a.oc channels, a box covers the CTA's 64)
        const cuuint64_t src_c = a.dw64 ? (cuuint64_t)a.oc : (cuuint64_t)a.ic;
        cuuint64_t dims[4] = {src_c, (cuuint64_t)a.iw, (cuuint64_t)a.ih, (cuuint64_t)images};
        cuuint64_t strides[3] = {src_c, (cuuint64_t)a.iw * src_c,
                                 (cuuint64_t)a.ih * a.iw * src_c};
        cuuint32_t box[4] = {64, (cuuint32_t)kRowCols, (cuuint32_t)pph, 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        CUresult r = api.tiled(
                &map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)src, dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return set_error(ST_RUNTIME, "cuTensorMapEncodeTiled(activation) failed: %d", (int)r);
        if (a.dw64) {
            map_b = map_a;  // unused: the kernel builds the filter tile itself
        } else {
        const cuuint64_t k_total = (cuuint64_t)a.kh * a.kw * a.ic;
        cuuint64_t bdims[2] = {k_total, (cuuint64_t)a.oc};
        cuuint64_t bstrides[1] = {k_total};
        cuuint32_t bbox[2] = {64, (cuuint32_t)pl.bn};
        cuuint32_t bestr[2] = {1, 1};
        r = api.tiled(
                &map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)flt, bdims, bstrides, bbox, bestr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return set_error(ST_RUNTIME, "cuTensorMapEncodeTiled(filter) failed: %d", (int)r);
        }
    } else if (a.ic == 16) {
        // one chunk: [row][column][16 bytes] is the tensor's own order, so a patch row is one
        // contiguous box row of ppw * 16 bytes
        cuuint64_t dims[3] = {(cuuint64_t)a.iw * 16, (cuuint64_t)a.ih, (cuuint64_t)images};
        cuuint64_t strides[2] = {(cuuint64_t)a.iw * 16, (cuuint64_t)a.ih * a.iw * 16};
        cuuint32_t box[3] = {(cuuint32_t)ppw * 16, (cuuint32_t)pph, 1};
        cuuint32_t estr[3] = {1, 1, 1};
        CUresult r = api.tiled(
                &map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, (void*)src, dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return set_error(ST_RUNTIME, "cuTensorMapEncodeTiled(activation) failed: %d", (int)r);
    } else {
        // NHWC seen as {16 channel bytes, W, H, N, C/16}: a box over all chunks arrives as
        // [chunk][row][column][16 bytes]
        cuuint64_t dims[5] = {16, (cuuint64_t)a.iw, (cuuint64_t)a.ih, (cuuint64_t)images,
                              (cuuint64_t)(a.ic / 16)};
        cuuint64_t strides[4] = {(cuuint64_t)a.ic, (cuuint64_t)a.iw * a.ic,
                                 (cuuint64_t)a.ih * a.iw * a.ic, 16};
        cuuint32_t box[5] = {16, (cuuint32_t)ppw, (cuuint32_t)pph, 1, (cuuint32_t)(a.ic / 16)};
        cuuint32_t estr[5] = {1, 1, 1, 1, 1};
        CUresult r = api.tiled(
                &map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 5, (void*)src, dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return set_error(ST_RUNTIME, "cuTensorMapEncodeTiled(activation) failed: %d", (int)r);
    }
    int b_single_load = 0;
    if (!pl.rows64) {
        const cuuint64_t k_total = (cuuint64_t)a.kh * a.kw * a.ic;
        const cuuint64_t kchunks = k_total / 16;
        CUresult r = CUDA_ERROR_INVALID_VALUE;
        if (kchunks <= 256) {
            // the packed filter [OC][K] seen as {16 bytes, OC rows (pitch K), K/16 blocks (pitch
            // 16)}: a box over all blocks arrives as [block][row][16 bytes], the operand layout
            cuuint64_t dims[3] = {16, (cuuint64_t)a.oc, kchunks};
            cuuint64_t strides[2] = {k_total, 16};
            cuuint32_t box[3] = {16, (cuuint32_t)pl.bn, (cuuint32_t)kchunks};
            cuuint32_t estr[3] = {1, 1, 1};
            r = api.tiled(
                    &map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, (void*)flt, dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            b_single_load = r == CUDA_SUCCESS;
        }
        if (r != CUDA_SUCCESS) {
            cuuint64_t dims[2] = {k_total, (cuuint64_t)a.oc};
            cuuint64_t strides[1] = {k_total};
            cuuint32_t box[2] = {16, (cuuint32_t)pl.bn};
            cuuint32_t estr[2] = {1, 1};
            r = api.tiled(
                    &map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)flt, dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        }
        if (r != CUDA_SUCCESS)
            return set_error(ST_RUNTIME, "cuTensorMapEncodeTiled(filter) failed: %d", (int)r);
    }

    PatchParams p;
    p.n = a.n;
    p.oh = a.oh;
    p.ow = a.ow;
    p.oc = a.oc;
    p.chunks = a.ic / 16;
    p.kh = a.kh;
    p.kw = a.kw;
    p.ph = a.ph;
    p.pw = a.pw;
    p.pph = pph;
    p.ppw = ppw;
    // MAX pooling 3x3 / 2 / pad 1 behind the ConvBias
    p.poh = (a.oh - 1) / 2 + 1;
    p.pow = (a.ow - 1) / 2 + 1;
    if (a.pool) {
        p.tiles_y = (p.poh + kPoolRows - 1) / kPoolRows;
        p.tiles_x = (p.pow + kPoolCols - 1) / kPoolCols;
    } else {
        p.tiles_y = (a.oh + kTH - 1) / kTH;
        p.tiles_x = (a.ow + kTW - 1) / kTW;
    }
    p.m_tiles = a.n * p.tiles_y * p.tiles_x;
    p.n_tiles = (a.oc + pl.bn - 1) / pl.bn;
    p.stages = pl.stages;
    p.a_stage_bytes = pl.a_stage_bytes;
    p.plane_stride = pl.plane_stride;
    p.a_tx_bytes = pl.rows64 ? pl.a_stage_bytes : p.chunks * pl.plane_stride;
    p.b_bytes = pl.b_bytes;
    p.b_single_load = b_single_load;
    p.a_flat16 = (!pl.rows64 && a.ic == 16) ? 1 : 0;
    p.mma_per_tap = a.ic == 16 ? 0 : a.ic / 32;
    p.a_lbo = a.ic == 16 ? 16 : p.plane_stride;
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
        fprintf(stderr, "%s: scales %g %g %g act %d z_mode %d verified requant: %d ops, %g + %.9g, short residual %g %g\n", "conv_patch",
                a.s_src, a.s_flt, a.s_dst, a.act, p.ep.z_mode, p.ep.fast_ops, p.ep.fast_mul, p.ep.fast_add,
                p.ep.z_fast_a,
                p.ep.z_fast_b);
    p.ep.acc_out = a.acc_out;
    p.overlap = tuning().overlap_loads;
    p.dw_flt = a.dw64 ? flt : nullptr;
    p.dw_pairs = a.dw64 == 2 ? 1 : 0;
    p.dst = dst;
    p.status = device_status_word(st);
    if (!p.status)
        return ST_MALLOC;
    // persistent grid: a multiple of the channel-slice count, at most what fits on the GPU
    int grid = sm_count() * pl.ctas_per_sm;
    grid = grid / p.n_tiles * p.n_tiles;
    if (grid < p.n_tiles)
        grid = p.n_tiles;
    const long long total = (long long)p.m_tiles * p.n_tiles;
    if (grid > total)
        grid = (int)total;
    int rc;
    const bool alone = pl.ctas_per_sm == 1;  // one CTA per SM: sixteen epilogue warps
    if (a.pool && a.kh == 4 && a.kw == 4 && a.ic == 16)
        rc = launch_patch<64, 4, 4, 1, 8, 0, 1>(map_a, map_b, p, pl.smem_bytes, grid, st);
    else if (a.pool)
        rc = launch_patch<64, 0, 0, 0, 8, 0, 1>(map_a, map_b, p, pl.smem_bytes, grid, st);
    else if (pl.rows64)
        rc = launch_patch<64, 3, 3, 4, 8, 1>(map_a, map_b, p, pl.smem_bytes, grid, st);
    else if (pl.bn == 64 && a.kh == 3 && a.kw == 3 && a.ic == 64 && !alone)
        rc = launch_patch<64, 3, 3, 4, 8>(map_a, map_b, p, pl.smem_bytes, grid, st);
    else if (pl.bn == 64 && a.kh == 4 && a.kw == 4 && a.ic == 16 && !alone)
        rc = launch_patch<64, 4, 4, 1, 8>(map_a, map_b, p, pl.smem_bytes, grid, st);
    else if (pl.bn == 128 && a.kh == 3 && a.kw == 3 && a.ic == 128 && alone)
        rc = launch_patch<128, 3, 3, 8, 16>(map_a, map_b, p, pl.smem_bytes, grid, st);
    else if (pl.bn == 64)
        // two 32-column chunks per lane quarter: eight epilogue warps at most
        rc = launch_patch<64, 0, 0, 0, 8>(map_a, map_b, p, pl.smem_bytes, grid, st);
    else
        rc = alone ? launch_patch<128, 0, 0, 0, 16>(map_a, map_b, p, pl.smem_bytes, grid, st)
                   : launch_patch<128, 0, 0, 0, 8>(map_a, map_b, p, pl.smem_bytes, grid, st);
    return rc;
}

// ---- depthwise 3x3 / stride 1 as 64-channel block-diagonal slices ----
namespace {
// the dense view the halo-patch kernel works on
ConvArgs dw_dense_view(const ConvArgs& a) {
    ConvArgs t = a;
    t.groups = 1;
    t.ic = 64;
    t.dw64 = 1;
    if (a.ic == 32) {
        // 32 channels: two horizontally adjacent pixels make one 64-byte "pixel"; with one
        // pixel of padding the pair x needs pairs x - 1 .. x + 1, a 3-wide filter again
        t.oc = 64;
        t.iw = a.iw / 2;
        t.ow = a.ow / 2;
        t.m = a.n * a.oh * t.ow;
        t.dw64 = 2;
    }
    return t;
}
}  // namespace

bool conv_patch_dw_supported(
        const ConvArgs& a, const int8_t* src, const int8_t* flt, const int8_t* dst,
        bool whatever_the_size) {
    if (a.groups != a.ic || a.oc != a.ic || a.kh != 3 || a.kw != 3)
        return false;
    // whole 64-channel slices, or 32 channels as pixel pairs (even widths, one pixel of padding)
    if (a.ic % 64 != 0 && !(a.ic == 32 && a.iw % 2 == 0 && a.ow == a.iw && a.pw == 1))
        return false;
    if (a.pool || a.acc_out)
        return false;
    const ConvArgs t = dw_dense_view(a);
    if (!conv_patch_supported(t, src, src, dst) || flt == nullptr)
        return false;
    if (whatever_the_size)
        return true;
    // A CTA builds its filter tile and sets up TMEM and barriers before its first patch, and a
    // partial 16 x 8 patch is paid for in full: the form is taken from four patches' worth of
    // real outputs per SM up. Measured against the CUDA-core kernel: 512 channels at 14 x 14
    // (77 % of the patch rows are outputs) 14.0 against 16.9 us at batch 64 and 26 against
    // 45 us at batch 256; 1024 channels at 7 x 7 (38 %) 14.7 against 14.4 us at batch 64 and
    // 22 against 33 us at batch 256.
    const long long tiles = (long long)t.n * ((t.oh + kTH - 1) / kTH) * ((t.ow + kTW - 1) / kTW) *
                            (t.oc / 64);
    return (double)tiles * conv_patch_efficiency(t) >= 4.0 * sm_count();
}

int launch_conv_patch_dw(
        const ConvArgs& a, const int8_t* src, const int8_t* flt, const int32_t* bias,
        const float* flt_scales, int8_t* dst, cudaStream_t st) {
    if (!conv_patch_dw_supported(a, src, flt, dst, true))
        return set_error(ST_NO_IMPLEMENT, "tensor-core depthwise ConvBias does not apply to this "
                                          "shape");
    return launch_conv_patch(dw_dense_view(a), src, flt, bias, flt_scales, dst, st);
}

}  // namespace mb200
