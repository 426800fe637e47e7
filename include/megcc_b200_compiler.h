/*
 * Compile side of megcc_b200 (libmegcc_b200_compiler.so): describes a static-shape
 * quantised network, asks the CUDA KernelGen pack for a kernel per operator, plans every
 * tensor into one device arena and writes the tinynn model.
 *
 * It stands in for the part of the reference's mgb-to-tinynn pipeline that follows the
 * importer: KernelMaterialization (compiler/lib/Dialect/Kernel/Transforms/
 * KernelMaterialization.cpp:136-158,212-276: operator -> TContext -> first available
 * KernelFunc), StaticMemoryPlanning (.../StaticMemoryPlanning.cpp:34-99: liveness ->
 * offsets into one buffer) and the tinynn exporter (compiler/lib/Target/TinyNN/
 * exporter.cpp:345-396,957-1001 and KernelExporter.cpp:15-66). The importer itself needs
 * MegEngine and is out of scope; operators are added through the calls below instead.
 *
 * All functions return a tensor id (>= 0) or a negative value on error;
 * mb200c_last_error() describes the failure. Host pointers throughout.
 */
#ifndef MEGCC_B200_COMPILER_H_
#define MEGCC_B200_COMPILER_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MB200C_API __attribute__((visibility("default")))

typedef struct mb200c_graph mb200c_graph;

MB200C_API mb200c_graph* mb200c_graph_create(const char* model_name);
MB200C_API void mb200c_graph_destroy(mb200c_graph* g);
MB200C_API const char* mb200c_last_error(void);

/* network input, qint8, model-visible layout NCHW; c/h/w are per image */
MB200C_API int mb200c_add_input(mb200c_graph* g, const char* name, int c, int h, int w, float scale);

/* ConvBias: operands src, filter, [bias], dst and attributes as
 * compiler/lib/Conversion/MGBToKernel/MGBToKernel.cpp:236-283 passes them.
 * flt: OIHW (groups == 1) or [G][OCpg][ICpg][KH][KW] int8; bias: [OC] int32 or NULL;
 * channel_scales: NULL (per-tensor flt_scale) or [OC] floats (extension).
 * nonline: "IDENTITY" | "RELU" | "H_SWISH". */
MB200C_API int mb200c_add_conv_bias(
        mb200c_graph* g, const char* name, int src, int oc, int kh, int kw, int stride, int pad,
        int groups, const char* nonline, const int8_t* flt, float flt_scale,
        const int32_t* bias, const float* channel_scales, float dst_scale);

/* A model compiled with --enable_nchw44 (compiler/tools/mgb-to-tinynn/mgb-to-tinynn.cpp:41-46;
 * the transform itself is MegEngine's, compiler/lib/Target/MGB/importer.cpp:1313-1367):
 * tensors are [N][C/4][H][W][4] and filters come in the layouts of
 * compiler/lib/KernelGen/BareMetal/ConvKernel.cpp:48-62,88-101. Such a model keeps its
 * visible layout: an input added here is read as NCHW44, every output with c % 4 == 0 is
 * handed back as NCHW44 (dims [N][C/4][H][W][4] in the model file), and the filters are
 * repacked by the Init step at load time; inside, activations are NHWC as always. */
MB200C_API int mb200c_add_input_nchw44(
        mb200c_graph* g, const char* name, int c, int h, int w, float scale);
/* flt44: dense [OC/4][IC/4][KH][KW][4][4] (groups == 1), channel-wise [G/4][1][1][KH][KW][4]
 * (groups == ic == oc), or, when src is an NCHW model input, the first-layer form
 * [OC/4][KH][KW][IC][4]. bias: [OC] in channel order (= [1][OC/4][1][1][4]). */
MB200C_API int mb200c_add_conv_bias_nchw44(
        mb200c_graph* g, const char* name, int src, int oc, int kh, int kw, int stride, int pad,
        int groups, const char* nonline, const int8_t* flt44, float flt_scale,
        const int32_t* bias, const float* channel_scales, float dst_scale);

/* MatrixMul + TypeCvt: C[batch][n] = requant(A[batch][K] x B[K][n]); A = tensor src with
 * h = w = 1 (K = its channels), b: [K][n] int8 row-major with per-tensor scale. The int32
 * product has scale src.scale * b_scale (one float multiplication, as MegEngine records it)
 * and is converted to qint8 at dst_scale by the TypeCvt rule
 * (compiler/lib/KernelGen/BareMetal/Typecvt.cpp:91-96). */
MB200C_API int mb200c_add_matmul(
        mb200c_graph* g, const char* name, int src, int n, const int8_t* b, float b_scale,
        float dst_scale);

/* mode: "MAX" | "AVERAGE" | "AVERAGE_COUNT_EXCLUDE_PADDING"; qint8 or fp32 by its input */
MB200C_API int mb200c_add_pooling(
        mb200c_graph* g, const char* name, int src, const char* mode, int window, int stride,
        int pad);

/* mode: "QADD" | "QFUSE_ADD_RELU" | "QMUL" | "QRELU" (b < 0 for QRELU) */
MB200C_API int mb200c_add_qelemwise(
        mb200c_graph* g, const char* name, const char* mode, int a, int b, float dst_scale);

/* ---- fp32 operators (the detector configuration). Tensors are fp32, model-visible layout
 * NCHW, NHWC inside the model. ---- */
MB200C_API int mb200c_add_input_f32(mb200c_graph* g, const char* name, int c, int h, int w);
/* ConvBias fp32: flt OIHW / [G][OCpg][ICpg][KH][KW] floats, bias [OC] floats or NULL.
 * nonline: "IDENTITY" | "RELU" | "SIGMOID" | "H_SWISH" (the reference's fp32 ConvBias modes,
 * compiler/lib/KernelGen/GeneralIntrinsic/ConvKernel/Fp32Im2col.cpp:130-134) or "SILU" (the
 * Elemwise SILU that follows a ConvBias in a YOLOX-style graph, folded in). z >= 0: a tensor
 * of the output's shape added after the activation (Elemwise ADD folded in), else -1. */
MB200C_API int mb200c_add_conv_f32(
        mb200c_graph* g, const char* name, int src, int oc, int kh, int kw, int stride, int pad,
        int groups, const char* nonline, const float* flt, const float* bias, int z);
/* MatrixMul fp32: C[batch][n] = A[batch][K] x B[K][n]; src has h = w = 1 */
MB200C_API int mb200c_add_matmul_f32(
        mb200c_graph* g, const char* name, int src, int n, const float* b);
/* Elemwise fp32, mode "RELU" | "SIGMOID" | "SILU" | "H_SWISH" | "EXP" (b = -1) or
 * "ADD" | "SUB" | "MUL" | "MAX" | "FUSE_ADD_RELU" (same-shape b) */
MB200C_API int mb200c_add_elemwise_f32(
        mb200c_graph* g, const char* name, const char* mode, int a, int b);
/* Concat along channels, 1..8 fp32 tensors of equal spatial extent */
MB200C_API int mb200c_add_concat(mb200c_graph* g, const char* name, const int* srcs, int nr);
/* Focus stem: the four stride-2 slices of the NCHW model input concatenated along channels
 * (in the reference: Subtensor views forwarded without a copy,
 * compiler/lib/Dialect/Kernel/Transforms/MemoryForwarding.cpp:36-85, plus a Concat); c_out >=
 * 4 * c, the extra channels are zeros */
MB200C_API int mb200c_add_focus(mb200c_graph* g, const char* name, int src, int c_out);
/* Resize NEAREST to oh x ow */
MB200C_API int mb200c_add_resize_nearest(mb200c_graph* g, const char* name, int src, int oh, int ow);

MB200C_API int mb200c_mark_output(mb200c_graph* g, int tensor);

/* Options:
 *   "fuse_conv_elemwise"  (on by default) a ConvBias without activation whose only consumer
 *                         is a QADD / QFUSE_ADD_RELU becomes one instruction (the z operand
 *                         slot of the reference's Conv2DKernel); results are bit-identical
 *                         to the two separate kernels (the MGB-level counterpart in the
 *                         reference is compiler/lib/Dialect/MGB/Transforms/KernelFuse.cpp
 *                         :41-80).
 *   "fuse_conv_pooling"   (off by default) a first-layer ConvBias (IDENTITY / RELU, at most
 *                         64 output channels) whose only consumer is a Pooling MAX 3x3 /
 *                         stride 2 / pad 1 becomes one instruction that never stores the
 *                         ConvBias result; bit-identical to the two kernels. Off because the
 *                         fused kernel measured slower than the pair it replaces.
 *   "bare_metal_model"    0 (default): CUDA_SM100 DeviceModels only. 1: a BARE_METAL
 *                         DeviceModel per batch size beside them (runtime/schema/model.fbs
 *                         :391 allows several), whose Oprs name the reference's own x86
 *                         kernels, one per operator, over NCHW tensors and the same weight
 *                         pool: the reference's C runtime and this runtime then execute one
 *                         artefact. 2: the BARE_METAL DeviceModels alone (the unmodified
 *                         reference runtime stops at a device value it does not know,
 *                         runtime/src/parse.c:78-99). For graphs of qint8 ConvBias with
 *                         per-tensor scales, Pooling and ElemwiseMultiType. */
MB200C_API int mb200c_set_option(mb200c_graph* g, const char* name, int value);

/* Compiles one DeviceModel (device CUDA_SM100) per batch size into a tinynn model.
 * The returned bytes belong to the graph and stay valid until it is destroyed or
 * compiled again. */
MB200C_API int mb200c_compile(
        mb200c_graph* g, const int* batches, int nr_batches, const uint8_t** bytes, size_t* len);

/* after mb200c_compile: newline-separated kernel symbols in kernel_id order */
MB200C_API const char* mb200c_kernel_symbols(mb200c_graph* g);
/* arena bytes the planner needed for batches[i], and the sum of tensor sizes it would
 * take without reuse */
MB200C_API size_t mb200c_arena_bytes(mb200c_graph* g, int batch_index);
MB200C_API size_t mb200c_unplanned_bytes(mb200c_graph* g, int batch_index);
/* Writes the generated sources the reference's exporter would: kernels.h, kernels.c
 * (tables + load_kernel_init_function) and one <symbol>.c per kernel. */
MB200C_API int mb200c_export_kernels(mb200c_graph* g, const char* dir);

/* KernelFunc probe used by the tests: 1 if the CUDA pack has an available ConvBias kernel
 * for this description, and its symbol. */
MB200C_API int mb200c_probe_conv_symbol(
        int ic, int oc, int h, int w, int k, int stride, int pad, int groups, const char* nonline,
        int with_bias, const char* format, char* symbol_out, size_t symbol_cap);

#ifdef __cplusplus
}
#endif
#endif /* MEGCC_B200_COMPILER_H_ */
