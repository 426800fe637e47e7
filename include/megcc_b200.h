/*
 * megcc_b200 operator-level C ABI (libmegcc_b200.so).
 *
 * These are the entry points that the host stubs emitted by the CUDA KernelGen arch
 * (GetKernelBody) call, one per reference kernel family. Every pointer is a DEVICE
 * pointer unless its name says host; `stream` is a cudaStream_t passed as void*.
 * All functions return a TinyNNStatus value (0 = TinyNN_SUCCESS,
 * runtime/src/tinynn.h:9-24 in the reference) and never throw or trap.
 *
 * Internal activation layout is NHWC int8 (channels innermost) so that one pixel's
 * channels are one contiguous TMA row; the model-visible layout stays the reference's
 * NCHW (compiler/lib/KernelGen/BareMetal/FormatHelper.cpp:18-22) and the *_nchw entry
 * points convert on the way in and out.
 *
 * Alignment contract. int8 tensors (activations, filters, z) may start at ANY byte: a
 * tensor that is not 16-byte aligned (a slice of a larger buffer) is computed by the general
 * CUDA-core kernels with byte loads, never by a vector or TMA path, and the results are the
 * same. int32 and float operands (bias, channel scales, int32 accumulators / products,
 * TypeCvt sources) must be 4-byte aligned as their type demands; a misaligned one is refused
 * with TinyNN_ERROR_INVALID_LAYOUT (12). Entry points that name a stricter rule (workspaces,
 * the fused operand z: 16 bytes) say so at their declaration. The tensor-core kernels
 * additionally want bias and channel scales 16-byte aligned and refuse them otherwise when
 * they were asked for by name (MB200_ALGO_UMMA / _PATCH); MB200_ALGO_AUTO falls back.
 *
 * Scale range. Results are bit-identical to the reference's x86 kernels for every finite
 * positive scale triple. The vector and tensor-core kernels divide by dst_scale with a
 * three-instruction sequence that is exact for 2^-100 <= src_scale * flt_scale <= 2^69,
 * 2^-100 <= dst_scale <= 2^100 and a ratio of the two within 2^-60 .. 2^60; outside that range MB200_ALGO_AUTO runs the general kernel
 * with the true division. One scale per output channel (flt_scales) must lie inside the
 * range by contract: the array is device memory and is not inspected by the host.
 */
#ifndef MEGCC_B200_H_
#define MEGCC_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MB200_API __attribute__((visibility("default")))

/* nonlineMode values of ConvBias (compiler/lib/KernelGen/BareMetal/Activation.cpp:9-42) */
enum { MB200_IDENTITY = 0, MB200_RELU = 1, MB200_H_SWISH = 2 };
/* Pooling modes (compiler/lib/KernelGen/BareMetal/Pooling.cpp:66-150) */
enum { MB200_POOL_MAX = 0, MB200_POOL_AVERAGE = 1, MB200_POOL_AVERAGE_COUNT_EXCLUDE_PADDING = 2 };
/* ElemwiseMultiType modes (compiler/lib/KernelGen/BareMetal/ElemwiseMultiType.cpp:26-56) */
enum { MB200_QADD = 0, MB200_QFUSE_ADD_RELU = 1, MB200_QMUL = 2, MB200_QRELU = 3 };
/* kernel choice for ConvBias: AUTO picks; DIRECT is the general CUDA-core kernel; UMMA the
 * tcgen05 implicit GEMM with TMA im2col loads; PATCH the tcgen05 halo-patch kernel (dense,
 * stride 1, or a depthwise 3x3 / stride 1 over whole 64-channel slices or over 32 channels,
 * which it runs with a block-diagonal filter). A named kernel that does not apply returns TinyNN_ERROR_NO_IMPLEMENT. */
enum { MB200_ALGO_AUTO = 0, MB200_ALGO_DIRECT = 1, MB200_ALGO_UMMA = 2, MB200_ALGO_PATCH = 3 };

/* The attributes the reference passes through TContext for a ConvBias
 * (kernel_h/w, stride_h/w, pad_h/w, dilate_h/w, sparse, nonlineMode:
 * compiler/lib/Conversion/MGBToKernel/MGBToKernelHelper.h:98-124) plus the extents its
 * kernel reads from the Tensor layouts (BareMetal/ConvKernel.cpp:287-301). */
typedef struct mb200_conv_param {
    int n, ic, ih, iw;
    int oc, kh, kw;
    int stride_h, stride_w, pad_h, pad_w, dilate_h, dilate_w;
    int groups;   /* 1 = DENSE, else GROUP (ic and oc are totals) */
    int nonline;  /* MB200_IDENTITY / MB200_RELU / MB200_H_SWISH */
    float src_scale, flt_scale, dst_scale;
} mb200_conv_param;

/* An ElemwiseMultiType step fused behind a ConvBias without activation: the int8 result of
 * the ConvBias (scale p->dst_scale, exactly what the stand-alone kernel would store) and the
 * int8 tensor z of the same NHWC shape go through kernel_elementwise_multitype_<MODE>
 * (compiler/lib/KernelGen/BareMetal/ElemwiseMultiType.cpp:38-46,158) with output scale
 * out_scale. Bit-identical to running the two kernels one after the other. */
typedef struct mb200_conv_fuse {
    const int8_t* z;
    int mode;        /* MB200_QADD or MB200_QFUSE_ADD_RELU */
    float z_scale;   /* scale of z */
    float out_scale; /* scale of the fused output */
} mb200_conv_fuse;

/* ---- library ---- */
MB200_API const char* mb200_version(void);
/* text of the last error raised on the calling thread ("" if none) */
MB200_API const char* mb200_last_error(void);
/* Kernel-selection switches for experiments and tests (the library's own choices are the
 * defaults): "conv_bn" 0|128|256, "conv_pair" 0|1, "conv_splitk" 0|2..4, "wide128" 1|0,
 * "patch_ctas" 0|1..3, "patch_alone" 0|1, "patch_plain" 0|1, "dw_out" 0|2|4,
 * "dw_one_output" 0|1, "fast_requant" 1|0, "debug" 0|1, "pdl" 1|0 (programmatic dependent
 * launch of consecutive kernels). Their initial values come from the
 * environment variables of the same meaning (MB200_CONV_BN, ...), read ONCE per process; no
 * launch consults the environment. Every setting yields bit-identical results. Process-wide,
 * not thread-safe against concurrent launches. */
MB200_API int mb200_set_option(const char* name, int value);
MB200_API int mb200_get_option(const char* name, int* value);
/* Reads and clears the status word that kernels launched on `stream` set when a bounded wait
 * ran out (0 = healthy; one word per device and stream). Synchronises `stream`. */
MB200_API int mb200_device_status(void* stream, int* status_host);

/* Self-test of the bounded device waits. Every wait inside the tensor-core kernels (on an
 * mbarrier that a TMA load or an MMA completes) has a time limit; when it runs out the kernel
 * records a code in the status word of its stream, lets the loads and MMAs it started
 * finish, frees its tensor memory and returns, so that the context stays usable and
 * LITE_wait can report TinyNN_ERROR_RUNTIME instead of hanging. This entry point makes that
 * happen on purpose without faulting anything: it launches the tensor-core ConvBias of `p`
 * (no bias, a shape the tensor-core kernel takes, >= 3 pipeline steps) with the limit
 * shortened to limit_cycles GPU clock cycles and with one pipeline stage per tile left
 * unfilled, so the MMA thread's wait for that stage expires. dst receives no defined result.
 * Afterwards mb200_device_status(stream) reports 0x102 (and clears it). The reference has no
 * counterpart (its runtime has no device and LITE_wait is a no-op,
 * runtime/src/lite/network.c:229-232). */
MB200_API int mb200_selftest_wait_expiry(
        const mb200_conv_param* p, const int8_t* src, const int8_t* flt_packed, int8_t* dst,
        long long limit_cycles, void* stream);

/* Measures the rate the tensor pipe of the current GPU sustains for tcgen05.mma kind::i8
 * (kind 0) or kind::tf32 (kind 1): one CTA per SM issues 40 000 MMAs of 128 x 256 x 32 bytes
 * on operands resident in shared memory. Result in tera-operations per second (2 per
 * multiply-accumulate). About 50 ms. Benchmarks use it as the roofline denominator where
 * no measured peak of that kind exists for the machine. */
MB200_API int mb200_measure_mma_rate(int kind, void* stream, double* tera_ops_per_second);

/* Tells the library that [base, base + bytes) is device memory the caller owns and that may
 * be READ anywhere inside (an arena). The tensor-core ConvBias kernels describe activations to
 * the TMA unit as tensors of at least 128 KiB; a smaller activation (batch 1 of a late layer)
 * takes them only when it lies in a registered range with enough bytes behind it, and the
 * general CUDA-core kernel otherwise. What is loaded from behind the activation is never
 * used. The runtime (LITE_*) registers its arenas itself (runtime/src/init.c:437-487 is where
 * the reference lays out its arena). Unregister before freeing the memory. */
MB200_API int mb200_register_readable_range(const void* base, size_t bytes);
MB200_API int mb200_unregister_readable_range(const void* base);

/* Parses a tinynn model (root table MegCC.Model, runtime/schema/model.fbs) the way the
 * runtime's loader does, without using a GPU, and writes a text summary into out.
 * Returns TinyNN_ERROR_MODEL_PARSE (7) for a truncated or malformed buffer. */
MB200_API int mb200_tinynn_describe(const void* model_mem, size_t size, char* out, size_t cap);

/* ---- ConvBias, qint8 x qint8 -> int32 -> qint8 ------------------------------------
 * Replaces kernel_conv2d_<k>x<k>_NCHW_{DENSE,GROUP}_p.._s.._d.._qsi8qsi8qsi32qsi8[_bias][_ACT]
 * (compiler/lib/KernelGen/BareMetal/ConvKernel.cpp:144-176, body :178-389). */

/* bytes of the K-major packed filter [OC][KH][KW][ICpg] that the kernels read */
MB200_API size_t mb200_conv_packed_filter_bytes(const mb200_conv_param* p);
/* OIHW / [G][OCpg][ICpg][KH][KW] -> packed. This is the Init step of the kernel
 * (the 3-phase init protocol of runtime/src/data_struct.h:135-142). */
MB200_API int mb200_conv_pack_filter(
        const mb200_conv_param* p, const int8_t* flt_oihw, int8_t* flt_packed, void* stream);
/* The same Init step for the filter of a model compiled with --enable_nchw44 (the layout
 * transform MegEngine's optimize_for_inference applies, compiler/lib/Target/MGB/importer.cpp
 * :1313-1367), layouts of compiler/lib/KernelGen/BareMetal/ConvKernel.cpp:48-62,88-101:
 *   form 0 dense        [OC/4][IC/4][KH][KW][4 ic][4 oc]
 *   form 1 channel-wise [G/4][1][1][KH][KW][4]
 *   form 2 first layer  [OC/4][KH][KW][IC][4 oc]   (NCHW input, NCHW44 output)
 * The result is exactly what mb200_conv_pack_filter (or mb200_conv_s2d_pack_filter, where
 * mb200_conv_s2d_supported(p)) gives for the same filter in OIHW, so the ConvBias entry
 * points are shared. Load-time only: it allocates and frees a scratch buffer of the filter's
 * size. */
MB200_API int mb200_conv_pack_filter_nchw44(
        const mb200_conv_param* p, int form, const int8_t* flt_nchw44, int8_t* flt_packed,
        void* stream);
/* src/dst NHWC. bias may be NULL. flt_scales: NULL = per-tensor p->flt_scale (all the
 * reference can express), else one float per output channel (extension).
 * src_is_nchw != 0 lets the first layer read the model input in place. */
MB200_API int mb200_conv_bias_qs8_nhwc(
        const mb200_conv_param* p, const int8_t* src, int src_is_nchw,
        const int8_t* flt_packed, const int32_t* bias, const float* flt_scales, int8_t* dst,
        int algo, void* stream);
/* mb200_conv_bias_qs8_nhwc with a fused elementwise step (fuse may be NULL: plain ConvBias) */
MB200_API int mb200_conv_bias_qs8_nhwc_fused(
        const mb200_conv_param* p, const int8_t* src, int src_is_nchw,
        const int8_t* flt_packed, const int32_t* bias, const float* flt_scales,
        const mb200_conv_fuse* fuse, int8_t* dst, int algo, void* stream);
/* First-layer form: stride 2 and at most 4 input channels run on the tensor cores after a
 * 2x2 space-to-depth step into `workspace` (device scratch, 16-byte aligned, at least
 * mb200_conv_s2d_workspace_bytes(p)). The filter must have been packed by
 * mb200_conv_s2d_pack_filter (mb200_conv_s2d_filter_bytes(p) bytes). Same operator and
 * results as mb200_conv_bias_qs8_nhwc. mb200_conv_s2d_supported(p) != 0 says the path
 * applies to p. */
MB200_API int mb200_conv_s2d_supported(const mb200_conv_param* p);
MB200_API size_t mb200_conv_s2d_filter_bytes(const mb200_conv_param* p);
MB200_API size_t mb200_conv_s2d_workspace_bytes(const mb200_conv_param* p);
MB200_API int mb200_conv_s2d_pack_filter(
        const mb200_conv_param* p, const int8_t* flt_oihw, int8_t* flt_s2d, void* stream);
MB200_API int mb200_conv_bias_qs8_s2d(
        const mb200_conv_param* p, const int8_t* src, int src_is_nchw, const int8_t* flt_s2d,
        const int32_t* bias, const float* flt_scales, int8_t* dst, void* workspace,
        size_t workspace_bytes, void* stream);
/* The same first-layer ConvBias followed by Pooling MAX, window 3x3, stride 2, pad 1
 * (compiler/lib/KernelGen/BareMetal/Pooling.cpp:66-150), as ONE kernel: dst is the pooled
 * tensor [n][(oh-1)/2+1][(ow-1)/2+1][oc] (NHWC), the ConvBias result itself is never stored.
 * Requantisation with positive scales and IDENTITY / RELU never decreases when the
 * accumulator grows, so the window maximum is taken on the int32 accumulators and the
 * result equals the two reference kernels run one after the other, bit for bit.
 * mb200_conv_s2d_pool_supported(p) != 0 says the form applies (the first-layer path, at most
 * 64 output channels in groups of 16, IDENTITY or RELU); all scales, per-channel ones
 * included, must be positive. */
MB200_API int mb200_conv_s2d_pool_supported(const mb200_conv_param* p);
MB200_API int mb200_conv_bias_pool_qs8_s2d(
        const mb200_conv_param* p, const int8_t* src, int src_is_nchw, const int8_t* flt_s2d,
        const int32_t* bias, const float* flt_scales, int8_t* dst, void* workspace,
        size_t workspace_bytes, void* stream);
/* Same operator in the reference's own layouts: src/dst NCHW, filter OIHW. Needs
 * mb200_conv_bias_qs8_nchw_workspace(p) bytes of device scratch (256-byte aligned). */
MB200_API size_t mb200_conv_bias_qs8_nchw_workspace(const mb200_conv_param* p);
MB200_API int mb200_conv_bias_qs8_nchw(
        const mb200_conv_param* p, const int8_t* src, const int8_t* flt_oihw,
        const int32_t* bias, const float* flt_scales, int8_t* dst, void* workspace,
        size_t workspace_bytes, int algo, void* stream);
/* The same operator for callers that cannot allocate device memory (a process whose own
 * pool already owns the whole device, or a loop that cannot afford the device-wide
 * synchronisation of cudaMalloc): this entry point has no counterpart in the reference.
 * The scratch mb200_conv_bias_qs8_nchw asks its caller for comes from a fixed array of
 * MB200_NOALLOC_SCRATCH_BYTES inside the library instead; the call makes no cudaMalloc,
 * cudaFree or other allocating call. Problems that need more scratch are refused with
 * TinyNN_ERROR_OUT_OF_RANGE (4) and a message naming both sizes. It runs the general
 * CUDA-core ConvBias kernel; results are identical to the other entry points.
 *  - The first call on each device resolves the array's device address; make that first call
 *    before any stream capture begins.
 *  - All calls on a device share the one array: two calls whose kernels overlap on the GPU
 *    (different streams without ordering between them) race. Calls on one stream are safe.
 *  - The array keeps the previous call's bytes; nothing depends on them, every byte read is
 *    written first within the same call. */
#define MB200_NOALLOC_SCRATCH_BYTES ((size_t)8 << 20)
MB200_API size_t mb200_conv_bias_qs8_nchw_noalloc_max_scratch(void);
MB200_API int mb200_conv_bias_qs8_nchw_noalloc(
        const mb200_conv_param* p, const int8_t* src, const int8_t* flt_oihw,
        const int32_t* bias, const float* flt_scales, int8_t* dst, void* stream);
/* int32 accumulators (bias added, before requantisation), NHWC; for accumulator parity */
MB200_API int mb200_conv_acc_qs8_nhwc(
        const mb200_conv_param* p, const int8_t* src, const int8_t* flt_packed,
        const int32_t* bias, int32_t* acc, void* stream);

/* Host only, no GPU needed. The tensor-core ConvBias epilogue may replace the reference's
 * three rounded float operations acc * src_scale * flt_scale / dst_scale
 * (compiler/lib/KernelGen/BareMetal/Activation.cpp:105-113) by a shorter form that ends in
 * one fused multiply-add: trunc(fma(f, mul, +-add)) with f = acc (1 operation), acc * src_scale
 * (2) or acc * src_scale * flt_scale (3); but only with constants for which the library has
 * shown that both are the same function of the int32 accumulator: both are monotonic
 * staircases, and they are compared on either side of every step of the reference's.
 * Returns the number of operations of the shortest form that passed, with its constants, or
 * 0 (and zeros) when none did, a scale is not positive or the activation is H_SWISH; the
 * kernels then keep the reference's operations. Cached per scale triple. */
MB200_API int mb200_requant_fast_constants(
        float src_scale, float flt_scale, float dst_scale, int nonline, float* mul, float* add);

/* ---- MatrixMul int8 x int8 -> int32 (C = A[M][K] * B[K][N], row-major), and the same with
 * the int32 product requantised to qint8 by the TypeCvt rule val * acc_scale / dst_scale
 * (compiler/lib/KernelGen/BareMetal/Typecvt.cpp:91-96). The reference has an int8 MatrixMul
 * only for Arm (compiler/lib/KernelGen/Arm/Arm64/MatMulKernel/Int8DotMatMulM8N12K4.cpp:20-31)
 * and none for x86 (BareMetal/MatrixMul.cpp:13-23 admits f32/f16), so the arithmetic follows
 * the exact integer definition. B is re-laid once to K-major rows (k*n bytes) by
 * mb200_matmul_pack_b, as a weight's Init step would. Runs on the tensor cores when
 * k % 64 == 0 and A holds at least 128 KiB. ---- */
MB200_API int mb200_matmul_pack_b(int k, int n, const int8_t* b, int8_t* b_packed, void* stream);
MB200_API int mb200_matmul_s8_s32(
        int m, int n, int k, const int8_t* a, const int8_t* b_packed, int32_t* c, void* stream);
MB200_API int mb200_matmul_s8_qs8(
        int m, int n, int k, const int8_t* a, const int8_t* b_packed, int8_t* c, float acc_scale,
        float dst_scale, void* stream);

/* ---- Pooling qint8 (kernel_pooling_<MODE>_NCHW_p.._s.._w.._qsi8qsi8,
 * compiler/lib/KernelGen/BareMetal/Pooling.cpp:166-273), NHWC in/out ---- */
MB200_API int mb200_pooling_qs8_nhwc(
        const int8_t* src, int8_t* dst, int mode, int n, int c, int ih, int iw, int window_h,
        int window_w, int stride_h, int stride_w, int pad_h, int pad_w, void* stream);

/* ---- Quantised elementwise (kernel_elementwise_multitype_<MODE>_qsi8qsi8qsi8,
 * compiler/lib/KernelGen/BareMetal/ElemwiseMultiType.cpp:102-213), same-shape operands.
 * b is ignored for MB200_QRELU. ---- */
MB200_API int mb200_qelemwise_qs8(
        const int8_t* a, const int8_t* b, int8_t* dst, int mode, size_t nr_elem, float scale_a,
        float scale_b, float scale_dst, void* stream);

/* The broadcast forms of the same kernel (the reference's fixture catalogue has a {2,3,4,5}
 * operand combined with {1,3,1,1} and with a scalar, compiler/test/kernel/opr/naive/
 * elemwise_multitype.cpp:33-62): element i of a meets b[(i / inner) % b_channels], or b[0]
 * when b_channels == 0. For an NCHW tensor and one value per channel inner = H * W; for NHWC
 * inner = 1. Modes QADD / QFUSE_ADD_RELU / QMUL. */
MB200_API int mb200_qelemwise_qs8_bcast(
        const int8_t* a, const int8_t* b, int8_t* dst, int mode, size_t nr_elem,
        size_t b_channels, size_t inner, float scale_a, float scale_b, float scale_dst,
        void* stream);

/* ---- TypeCvt between fp32 and qsi8, the rule of the reference's x86 build: these dtype pairs
 * resolve to GI_kernel_typecvt_* there (compiler/lib/KernelGen/GeneralIntrinsic/Typecvt.cpp
 * :176-190,258-267), which multiplies by scale = src_scale / dst_scale (one float division on
 * the host; the scale of the FLOAT side counts as 1 whatever is passed, :56-69) and stores
 * clamp(round(v * scale)), half away from zero; qsi8 -> fp32 is v * scale. ---- */
MB200_API int mb200_typecvt_f32_qs8(
        const float* src, int8_t* dst, size_t nr_elem, float src_scale, float dst_scale,
        void* stream);
MB200_API int mb200_typecvt_qs8_f32(
        const int8_t* src, float* dst, size_t nr_elem, float src_scale, float dst_scale,
        void* stream);

/* ---- TypeCvt qsi32 -> qsi8 (kernel_typecvt_qsi32qsi8,
 * compiler/lib/KernelGen/BareMetal/Typecvt.cpp:43-106) ---- */
MB200_API int mb200_typecvt_qs32_qs8(
        const int32_t* src, int8_t* dst, size_t nr_elem, float src_scale, float dst_scale,
        void* stream);

/* ---- Layout transforms between the model-visible NCHW and the internal NHWC
 * (the reference's Relayout/Dimshuffle, compiler/lib/KernelGen/BareMetal/Relayout.cpp:13-23) */
MB200_API int mb200_relayout_nchw_to_nhwc_s8(
        const int8_t* src, int8_t* dst, int n, int c, int h, int w, void* stream);
MB200_API int mb200_relayout_nhwc_to_nchw_s8(
        const int8_t* src, int8_t* dst, int n, int c, int h, int w, void* stream);

/* ======================================================================================
 * fp32 path (the detector configuration and the fp32 MatrixMul sweep). NHWC fp32 tensors,
 * 4-byte aligned at least; the vector and tensor-core paths want 16 bytes and fall back to
 * scalar kernels otherwise. Results agree with the reference's x86 kernels within 1e-4
 * relative / 1e-5 absolute (fp32 sums in a different order), not bit for bit.
 * ====================================================================================== */

/* nonlineMode of an fp32 ConvBias. The reference's fp32 ConvBias kernels take IDENTITY / RELU /
 * SIGMOID / H_SWISH (compiler/lib/KernelGen/GeneralIntrinsic/ConvKernel/Fp32Im2col.cpp:130-134);
 * SILU is the Elemwise kernel that follows a ConvBias in a YOLOX-style graph
 * (BareMetal/ElemwiseKernel.cpp:52-53), folded into the epilogue here. */
enum { MB200_F32_IDENTITY = 0, MB200_F32_RELU = 1, MB200_F32_H_SWISH = 2, MB200_F32_SIGMOID = 3,
       MB200_F32_SILU = 4 };
/* Elemwise modes (compiler/lib/KernelGen/BareMetal/ElemwiseKernel.cpp:20-120); unary below 16 */
enum { MB200_ELEM_RELU = 0, MB200_ELEM_SIGMOID = 1, MB200_ELEM_SILU = 2, MB200_ELEM_H_SWISH = 3,
       MB200_ELEM_EXP = 4, MB200_ELEM_ADD = 16, MB200_ELEM_SUB = 17, MB200_ELEM_MUL = 18,
       MB200_ELEM_MAX = 19, MB200_ELEM_FUSE_ADD_RELU = 20 };

typedef struct mb200_conv_f32_param {
    int n, ic, ih, iw;
    int oc, kh, kw;
    int stride_h, stride_w, pad_h, pad_w;
    int groups;  /* 1 = DENSE */
    int nonline; /* MB200_F32_* */
} mb200_conv_f32_param;

/* ---- ConvBias fp32 (replaces GI_kernel_conv2d_im2col_<k>x<k>_NCHW_DENSE_..._f32,
 * compiler/lib/KernelGen/GeneralIntrinsic/ConvKernel/Fp32Im2col.cpp:88-120, body :198-217).
 * The Init step (mb200_conv_f32_pack_filter) turns the OIHW filter into the K-major form
 * [OC][KH][KW][ICpg] followed, for dense filters whose channel count fills whole TMA rows (16
 * or a multiple of 32), by its two tf32 planes for the tensor cores. The activation is split
 * into its planes in shared memory, so the ConvBias needs no scratch:
 * mb200_conv_f32_workspace_bytes(p) answers 0 and `workspace` may be NULL (both are kept so
 * that callers written against earlier versions keep working).
 *   bias   [OC] floats or NULL
 *   z      optional NHWC tensor of the output's shape added AFTER the activation (the shortcut
 *          of a bottleneck block: an Elemwise ADD folded into the epilogue), or NULL
 *   dst_pitch  floats between consecutive output pixels; 0 = oc. A larger pitch lets the
 *          ConvBias write its channel slice of a wider buffer (a Concat without a copy).
 *   algo   MB200_ALGO_AUTO / MB200_ALGO_DIRECT (CUDA cores) / MB200_ALGO_UMMA (tensor cores) */
MB200_API size_t mb200_conv_f32_packed_filter_bytes(const mb200_conv_f32_param* p);
MB200_API int mb200_conv_f32_pack_filter(
        const mb200_conv_f32_param* p, const float* flt_oihw, float* flt_packed, void* stream);
MB200_API size_t mb200_conv_f32_workspace_bytes(const mb200_conv_f32_param* p);
MB200_API int mb200_conv_bias_f32_nhwc(
        const mb200_conv_f32_param* p, const float* src, const float* flt_packed,
        const float* bias, const float* z, float* dst, long long dst_pitch, void* workspace,
        size_t workspace_bytes, int algo, void* stream);

/* ---- MatrixMul fp32, C[M][N] = A[M][K] * B[K][N], row-major (replaces
 * GI_kernel_fp32_matmul_4x12_nn, compiler/lib/KernelGen/GeneralIntrinsic/MatMulKernel/
 * Fp32MatMulM4N12.cpp:8-160). B is prepared once by mb200_matmul_f32_pack_b into
 * mb200_matmul_f32_packed_b_bytes(k, n) bytes; the product needs no scratch
 * (mb200_matmul_f32_workspace_bytes answers 0). Tensor cores (three tf32 passes)
 * when k % 32 == 0 (or k == 16) and A holds at least 128 KiB. */
MB200_API size_t mb200_matmul_f32_packed_b_bytes(int k, int n);
MB200_API int mb200_matmul_f32_pack_b(int k, int n, const float* b, float* b_packed, void* stream);
MB200_API size_t mb200_matmul_f32_workspace_bytes(int m, int k);
MB200_API int mb200_matmul_f32(
        int m, int n, int k, const float* a, const float* b_packed, float* c, void* workspace,
        size_t workspace_bytes, void* stream);

/* ---- Elemwise fp32, same-shape operands (b ignored for unary modes) ---- */
MB200_API int mb200_elemwise_f32(
        int mode, const float* a, const float* b, float* dst, size_t nr_elem, void* stream);

/* ---- Concat along channels of NHWC tensors with the same pixel count (kernel_concat_*,
 * compiler/lib/KernelGen/BareMetal/Concat.cpp:23-78); at most 8 inputs ---- */
MB200_API int mb200_concat_f32_nhwc(
        const float* const* srcs_host_array, const int* channels_host_array, int nr_inputs,
        float* dst, size_t pixels, void* stream);

/* ---- Resize NEAREST (kernel_resize_linear_NCHW_NEAREST_f32: ih = min((int)(oh / scale),
 * IH - 1), compiler/lib/KernelGen/Common/Resize.h:155-156), NHWC ---- */
MB200_API int mb200_resize_nearest_f32_nhwc(
        const float* src, float* dst, int n, int c, int ih, int iw, int oh, int ow, void* stream);

/* ---- Pooling fp32 (kernel_pooling_<MODE>_NCHW_..._f32f32,
 * compiler/lib/KernelGen/BareMetal/Pooling.cpp:166-273), NHWC, modes as MB200_POOL_* ---- */
MB200_API int mb200_pooling_f32_nhwc(
        const float* src, float* dst, int mode, int n, int c, int ih, int iw, int window_h,
        int window_w, int stride_h, int stride_w, int pad_h, int pad_w, void* stream);

/* ---- Focus stem: the four stride-2 slices of an NCHW image concatenated along channels in
 * the order (even rows, even cols), (odd, even), (even, odd), (odd, odd), written as an NHWC
 * tensor [N][H/2][W/2][c_out] with c_out >= 4 * c (extra channels zero, so that the first
 * ConvBias reads whole TMA rows). In the reference these are four Subtensor views turned into
 * zero-copy MemForward instructions (compiler/lib/Dialect/Kernel/Transforms/
 * MemoryForwarding.cpp:36-85, runtime/src/vm/memforward.c:41-51) feeding a Concat. ---- */
MB200_API int mb200_focus_f32(
        const float* src_nchw, float* dst_nhwc, int n, int c, int h, int w, int c_out,
        void* stream);

/* ---- model-boundary layout transforms, fp32 ---- */
MB200_API int mb200_relayout_nchw_to_nhwc_f32(
        const float* src, float* dst, int n, int c, int h, int w, void* stream);
MB200_API int mb200_relayout_nhwc_to_nchw_f32(
        const float* src, float* dst, int n, int c, int h, int w, void* stream);

/* ---- NCHW44 activations [N][C/4][H][W][4] (compiler/lib/KernelGen/BareMetal/FormatHelper.cpp
 * :23-26) <-> the internal NHWC, at the boundary of a model compiled with --enable_nchw44;
 * c % 4 == 0, 4-byte aligned tensors ---- */
MB200_API int mb200_relayout_nchw44_to_nhwc_s8(
        const int8_t* src, int8_t* dst, int n, int c, int h, int w, void* stream);
MB200_API int mb200_relayout_nhwc_to_nchw44_s8(
        const int8_t* src, int8_t* dst, int n, int c, int h, int w, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MEGCC_B200_H_ */
