#include "cuda_kernel_pack.h"

#include "../csrc/conv_s2d_geom.h"

#include <cmath>
#include <cstdio>
#include <sstream>

using namespace megcc;
using namespace megcc::KernelGen;
using namespace megcc::KernelGen::Cuda;

namespace {

bool is_quant(const std::string& dtype, int bits) {
    const std::string prefix = "qsi" + std::to_string(bits);
    return dtype.compare(0, prefix.size(), prefix) == 0 &&
           (dtype.size() == prefix.size() || dtype[prefix.size()] == '<');
}

// dtype string without its "<...>" parameter, as the reference's symbols spell it
// (compiler/lib/KernelGen/Utils/SymbolHelper.h:9-24)
std::string bare_dtype(const std::string& dtype) {
    const auto p = dtype.find('<');
    return p == std::string::npos ? dtype : dtype.substr(0, p);
}

std::string io_str(TContext* ctx) {
    std::string s;
    const int n = ctx->getAttrInt("nr_operands");
    for (int i = 0; i < n; ++i)
        s += bare_dtype(ctx->getAttrOprand("operand:" + std::to_string(i)).dtype);
    return s;
}

CCOperand last_operand(TContext* ctx) {
    return ctx->getAttrOprand("operand:" + std::to_string(ctx->getAttrInt("nr_operands") - 1));
}

// bias present iff there are more than 3 operands and operand 2 has a shape
// (compiler/lib/KernelGen/Common/ConvKernel.h:10-21)
bool has_bias(TContext* ctx) {
    return ctx->getAttrInt("nr_operands") > 3 &&
           ctx->getAttrOprand("operand:2").shape.size() > 0;
}

bool channel_broadcast_bias(TContext* ctx) {
    const CCOperand b = ctx->getAttrOprand("operand:2");
    if (b.shape.size() == 1)
        return true;
    if (b.shape.size() == 5)  // NCHW44: [1][C/4][1][1][4], the channels in order
        return b.shape[0] == 1 && b.shape[2] == 1 && b.shape[3] == 1 && b.shape[4] == 4;
    return b.shape.size() == 4 && b.shape[0] == 1 && b.shape[2] == 1 && b.shape[3] == 1;
}

// Filter layout of a ConvBias: 0 OIHW / GOIHW; for format NCHW44 (the filters of a model
// compiled with --enable_nchw44, compiler/lib/KernelGen/BareMetal/ConvKernel.cpp:48-62,88-101)
// 1 dense [OC/4][IC/4][KH][KW][4][4], 2 channel-wise [G/4][1][1][KH][KW][4], 3 first layer
// [OC/4][KH][KW][IC][4] (NCHW input: FormatHelper.cpp's "NCHW_NCHW44"); -1 not one of them
int filter_form(TContext* ctx) {
    const std::string format = ctx->getAttrStr("format");
    if (format == "NCHW")
        return 0;
    if (format != "NCHW44")
        return -1;
    const CCOperand src = ctx->getAttrOprand("operand:0");
    const CCOperand flt = ctx->getAttrOprand("operand:1");
    const size_t kh = ctx->getAttrUInt("kernel_h"), kw = ctx->getAttrUInt("kernel_w");
    const bool dense = ctx->getAttrStr("sparse") == "DENSE";
    if (src.shape.size() == 4)
        return dense && flt.shape.size() == 5 && flt.shape[1] == kh && flt.shape[2] == kw &&
                               flt.shape[3] == src.shape[1] && flt.shape[4] == 4
                       ? 3
                       : -1;
    if (src.shape.size() != 5 || src.shape[4] != 4 || flt.shape.size() != 6 || flt.shape[5] != 4)
        return -1;
    if (dense)
        return flt.shape[1] == src.shape[1] && flt.shape[2] == kh && flt.shape[3] == kw &&
                               flt.shape[4] == 4
                       ? 1
                       : -1;
    return flt.shape[0] == src.shape[1] && flt.shape[1] == 1 && flt.shape[2] == 1 &&
                           flt.shape[3] == kh && flt.shape[4] == kw
                   ? 2
                   : -1;
}

const char* filter_form_token(int form) {
    static const char* names[] = {"NHWC", "NHWC44D", "NHWC44C", "NHWC44H"};
    return names[form];
}

// "" unless the operator carries a fused ElemwiseMultiType step (5 operands: src, filter,
// bias, z, dst)
std::string fuse_mode(TContext* ctx) {
    return ctx->haveAttr("fuse_elemwise_mode") ? ctx->getAttrStr("fuse_elemwise_mode") : "";
}

// "" unless the MAX pooling 3x3 / stride 2 / pad 1 behind the ConvBias is part of the operator
std::string fuse_pool(TContext* ctx) {
    return ctx->haveAttr("fuse_pooling") ? ctx->getAttrStr("fuse_pooling") : "";
}

std::string nonline(TContext* ctx) {
    return ctx->haveAttr("nonlineMode") ? ctx->getAttrStr("nonlineMode") : "IDENTITY";
}

int nonline_code(const std::string& m) {
    return m == "RELU" ? 1 : m == "H_SWISH" ? 2 : 0;
}

struct Subst {
    std::string text;
    Subst& set(const std::string& key, const std::string& value) {
        const std::string pat = "${" + key + "}";
        for (size_t p = text.find(pat); p != std::string::npos; p = text.find(pat, p))
            text.replace(p, pat.size(), value), p += value.size();
        return *this;
    }
    Subst& set(const std::string& key, long long v) { return set(key, std::to_string(v)); }
};

}  // namespace

std::string Cuda::GenStubPrologue() {
    return "#include \"megcc_b200_runtime.h\"\n#include \"megcc_b200.h\"\n";
}

// ------------------------------------------------------------------------------------------
// ConvBias
// ------------------------------------------------------------------------------------------
bool ConvBiasQS8::IsAvailable(TContext* ctx) const {
    if (ctx->getAttrStr("mode") != "CROSS_CORRELATION")
        return false;
    if (ctx->getAttrInt("nr_operands") < 3)
        return false;
    const CCOperand src = ctx->getAttrOprand("operand:0");
    const CCOperand flt = ctx->getAttrOprand("operand:1");
    const CCOperand dst = last_operand(ctx);
    if (!is_quant(src.dtype, 8) || !is_quant(flt.dtype, 8) || !is_quant(dst.dtype, 8))
        return false;
    // NCHW, or NCHW44 with the filter repacked at load time (the tensors of such a model are
    // converted to the internal NHWC at its boundary)
    const int form = filter_form(ctx);
    if (form < 0 || (form == 0 && src.shape.size() != 4))
        return false;
    const std::string sparse = ctx->getAttrStr("sparse");
    if (sparse != "DENSE" && sparse != "GROUP")
        return false;
    const std::string act = nonline(ctx);
    if (act != "IDENTITY" && act != "RELU" && act != "H_SWISH")
        return false;
    const std::string fm = fuse_mode(ctx);
    if (!fm.empty()) {
        // fused residual step: needs the z operand, no activation on the ConvBias itself
        if (ctx->getAttrInt("nr_operands") != 5 || act != "IDENTITY" ||
            (fm != "QADD" && fm != "QFUSE_ADD_RELU"))
            return false;
        const CCOperand z = ctx->getAttrOprand("operand:3");
        if (!is_quant(z.dtype, 8) || z.shape != dst.shape)
            return false;
    } else if (ctx->getAttrInt("nr_operands") > 4) {
        return false;
    }
    if (has_bias(ctx)) {
        const CCOperand bias = ctx->getAttrOprand("operand:2");
        if (!is_quant(bias.dtype, 32) || !channel_broadcast_bias(ctx))
            return false;
        // same scale consistency rule as the reference (ConvKernel.cpp:37-42)
        if (std::fabs(src.scale * flt.scale - bias.scale) >= 1e-5)
            return false;
    }
    const std::string fp = fuse_pool(ctx);
    if (!fp.empty()) {
        // ConvBias + MAX pooling: only the first-layer form (NCHW input, few channels,
        // stride 2) with at most 64 output channels has the pooled epilogue, and taking the
        // maximum before the requantisation needs that to be non-decreasing
        if (fp != "MAX_3x3_s2x2_p1x1" || !fm.empty() || act == "H_SWISH" ||
            src.shape.size() != 4 || sparse != "DENSE" || ctx->getAttrUInt("dilate_h") != 1 ||
            ctx->getAttrUInt("dilate_w") != 1 || !(src.scale > 0) || !(flt.scale > 0) ||
            !(dst.scale > 0))
            return false;
        const int oc = (int)(dst.shape.size() == 5 ? dst.shape[1] * 4 : dst.shape[1]);
        const mb200::S2dGeom g = mb200::s2d_geometry(
                (int)src.shape[0], (int)src.shape[1], (int)src.shape[2], (int)src.shape[3], oc,
                (int)ctx->getAttrUInt("kernel_h"), (int)ctx->getAttrUInt("kernel_w"),
                (int)ctx->getAttrUInt("stride_h"), (int)ctx->getAttrUInt("stride_w"),
                (int)ctx->getAttrUInt("pad_h"), (int)ctx->getAttrUInt("pad_w"), 1, 1, 1);
        if (!mb200::s2d_pool_fusable(g, oc))
            return false;
    }
    return true;
}

std::string ConvBiasQS8::GetKernelSymbol(TContext* ctx) const {
    if (!ctx)  // the dispatcher probes symbols with a null context (KernelGen.cpp:49,108)
        return "cuda_sm100_conv2d";
    std::stringstream ss;
    ss << "cuda_sm100_conv2d_" << ctx->getAttrUInt("kernel_h") << "x"
       << ctx->getAttrUInt("kernel_w") << "_" << filter_form_token(filter_form(ctx)) << "_"
       << ctx->getAttrStr("sparse") << "_p"
       << ctx->getAttrUInt("pad_h") << "x" << ctx->getAttrUInt("pad_w") << "_s"
       << ctx->getAttrUInt("stride_h") << "x" << ctx->getAttrUInt("stride_w") << "_d"
       << ctx->getAttrUInt("dilate_h") << "x" << ctx->getAttrUInt("dilate_w") << "_"
       << io_str(ctx);
    if (has_bias(ctx))
        ss << "_bias";
    if (nonline(ctx) != "IDENTITY")
        ss << "_" << nonline(ctx);
    if (!fuse_mode(ctx).empty())
        ss << "_z_" << fuse_mode(ctx);
    if (!fuse_pool(ctx).empty())
        ss << "_pool_MAX3x3s2p1";
    return ss.str();
}

std::string ConvBiasQS8::GetKernelBody(TContext* ctx) const {
    Subst s{R"(
${prologue}
/* dims are the logical NCHW extents; strides say the buffer is NHWC */
TinyNNStatus ${signature} {
    const Tensor* src = inputs[0];
    const Tensor* flt = inputs[1];
    const Tensor* dst = outputs[0];
    mb200_conv_param p;
    p.n = src->layout.dims[0];
    p.ic = src->layout.dims[1];
    p.ih = src->layout.dims[2];
    p.iw = src->layout.dims[3];
    p.oc = dst->layout.dims[1];
    p.kh = ${kh}; p.kw = ${kw};
    p.stride_h = ${sh}; p.stride_w = ${sw};
    p.pad_h = ${ph}; p.pad_w = ${pw};
    p.dilate_h = ${dh}; p.dilate_w = ${dw};
    p.groups = ${dense} ? 1 : (int)flt->layout.dims[0] * ${group_block};
    p.nonline = ${nonline};
    p.src_scale = src->dtype.param.scale;
    p.flt_scale = flt->dtype.param.scale;
    p.dst_scale = dst->dtype.param.scale;
    const int src_is_nchw = src->layout.format == TinyNN_NCHW;
    const int32_t* bias = ${has_bias} ? (const int32_t*)inputs[2]->ptr : 0;
    /* inputs: src, filter, [bias], [channel scales], [z, mid scale] */
    const int nr_plain = nr_input - ${fused} * 2;
    const float* ch_scales = nr_plain > ${scale_idx} ? (const float*)inputs[${scale_idx}]->ptr : 0;
    if (${fused}) {
        mb200_conv_fuse fuse;
        fuse.z = (const int8_t*)inputs[nr_input - 2]->ptr;
        fuse.mode = ${fuse_code};
        fuse.z_scale = inputs[nr_input - 2]->dtype.param.scale;
        fuse.out_scale = dst->dtype.param.scale;
        /* the ConvBias result keeps its own scale; it travels as the dtype scale of a
         * 1-element weight, the last input */
        p.dst_scale = inputs[nr_input - 1]->dtype.param.scale;
        return (TinyNNStatus)mb200_conv_bias_qs8_nhwc_fused(
                &p, (const int8_t*)src->ptr, src_is_nchw, (const int8_t*)flt->ptr, bias, ch_scales,
                &fuse, (int8_t*)dst->ptr, MB200_ALGO_AUTO, mb200_opt_stream(opt));
    }
    if (${pooled}) {
        /* dst is the tensor behind the MAX pooling 3x3 / 2 / pad 1 that follows */
        return (TinyNNStatus)mb200_conv_bias_pool_qs8_s2d(
                &p, (const int8_t*)src->ptr, src_is_nchw, (const int8_t*)flt->ptr, bias, ch_scales,
                (int8_t*)dst->ptr, workspace->ptr, workspace->size, mb200_opt_stream(opt));
    }
    if (mb200_conv_s2d_supported(&p)) {
        /* first-layer form; the filter was packed for it by the init function below */
        return (TinyNNStatus)mb200_conv_bias_qs8_s2d(
                &p, (const int8_t*)src->ptr, src_is_nchw, (const int8_t*)flt->ptr, bias, ch_scales,
                (int8_t*)dst->ptr, workspace->ptr, workspace->size, mb200_opt_stream(opt));
    }
    return (TinyNNStatus)mb200_conv_bias_qs8_nhwc(
            &p, (const int8_t*)src->ptr, src_is_nchw, (const int8_t*)flt->ptr, bias, ch_scales,
            (int8_t*)dst->ptr, MB200_ALGO_AUTO, mb200_opt_stream(opt));
}
)"};
    const bool bias = has_bias(ctx);
    s.set("prologue", GenStubPrologue())
            .set("signature", GetKernelSignature(ctx))
            .set("kh", ctx->getAttrUInt("kernel_h"))
            .set("kw", ctx->getAttrUInt("kernel_w"))
            .set("sh", ctx->getAttrUInt("stride_h"))
            .set("sw", ctx->getAttrUInt("stride_w"))
            .set("ph", ctx->getAttrUInt("pad_h"))
            .set("pw", ctx->getAttrUInt("pad_w"))
            .set("dh", ctx->getAttrUInt("dilate_h"))
            .set("dw", ctx->getAttrUInt("dilate_w"))
            .set("dense", ctx->getAttrStr("sparse") == "DENSE" ? 1 : 0)
            .set("group_block", filter_form(ctx) ? 4 : 1)
            .set("nonline", nonline_code(nonline(ctx)))
            .set("has_bias", bias ? 1 : 0)
            .set("scale_idx", bias ? 3 : 2);
    const std::string fm = fuse_mode(ctx);
    s.set("fused", fm.empty() ? 0 : 1).set("fuse_code", fm == "QADD" ? 0 : 1);
    s.set("pooled", fuse_pool(ctx).empty() ? 0 : 1);
    return s.text;
}

// Init: the filter weight is re-laid from OIHW / [G][OCpg][ICpg][KH][KW] to the K-major
// [OC][KH][KW][ICpg] the kernels read. Follows the 3-phase protocol of
// runtime/src/data_struct.h:135-142 (count, describe, fill) and keeps the weight's name
// pointer, which the runtime matches on (runtime/src/init.c:64,192).
std::string ConvBiasQS8::GetInitBody(TContext* ctx) const {
    Subst s{R"(
${prologue}
static void ${symbol}_param(Tensor** inputs, mb200_conv_param* p) {
    const Tensor* src = inputs[0];
    const Layout* l = &inputs[1]->layout;
    const int grouped = !${dense};
    p->n = src->layout.dims[0];
    p->ic = src->layout.dims[1];
    p->ih = src->layout.dims[2];
    p->iw = src->layout.dims[3];
    if (${form}) { /* NCHW44 layouts count blocks of four output channels (or groups) */
        p->groups = grouped ? (int)l->dims[0] * 4 : 1;
        p->oc = (int)l->dims[0] * 4;
    } else {
        p->groups = grouped ? (int)l->dims[0] : 1;
        p->oc = grouped ? (int)(l->dims[0] * l->dims[1]) : (int)l->dims[0];
    }
    p->kh = ${kh}; p->kw = ${kw};
    p->stride_h = ${sh}; p->stride_w = ${sw};
    p->pad_h = ${ph}; p->pad_w = ${pw};
    p->dilate_h = ${dh}; p->dilate_w = ${dw};
    p->nonline = 0;
    p->src_scale = p->flt_scale = p->dst_scale = 1.f;
}
TinyNNStatus ${signature} {
    Tensor* in_weights = inputs[1];
    mb200_conv_param p;
    ${symbol}_param(inputs, &p);
    const int s2d = mb200_conv_s2d_supported(&p);
    if (out_weights == 0 && nr_out_weight != 0) {
        *nr_out_weight = 1;
        return TinyNN_SUCCESS;
    }
    if (out_weights != 0 && nr_out_weight == 0) {
        out_weights->layout = in_weights->layout;
        if (s2d) { /* a flat byte buffer of the space-to-depth packing */
            out_weights->layout.nr_dim = 1;
            out_weights->layout.dims[0] = (uint32_t)mb200_conv_s2d_filter_bytes(&p);
            out_weights->layout.stride[0] = 1;
        }
        out_weights->dtype = in_weights->dtype;
        out_weights->name = in_weights->name;
        return TinyNN_SUCCESS;
    }
    if (${form}) /* from the NCHW44 layout straight to whichever packing the kernel reads */
        return (TinyNNStatus)mb200_conv_pack_filter_nchw44(
                &p, ${form} - 1, (const int8_t*)in_weights->ptr, (int8_t*)out_weights->ptr,
                mb200_opt_stream(opt));
    if (s2d)
        return (TinyNNStatus)mb200_conv_s2d_pack_filter(
                &p, (const int8_t*)in_weights->ptr, (int8_t*)out_weights->ptr,
                mb200_opt_stream(opt));
    return (TinyNNStatus)mb200_conv_pack_filter(
            &p, (const int8_t*)in_weights->ptr, (int8_t*)out_weights->ptr, mb200_opt_stream(opt));
}
)"};
    s.set("prologue", GenStubPrologue())
            .set("signature", GetInitSignature(ctx))
            .set("symbol", GetKernelSymbol(ctx))
            .set("form", filter_form(ctx))
            .set("dense", ctx->getAttrStr("sparse") == "DENSE" ? 1 : 0)
            .set("kh", ctx->getAttrUInt("kernel_h"))
            .set("kw", ctx->getAttrUInt("kernel_w"))
            .set("sh", ctx->getAttrUInt("stride_h"))
            .set("sw", ctx->getAttrUInt("stride_w"))
            .set("ph", ctx->getAttrUInt("pad_h"))
            .set("pw", ctx->getAttrUInt("pad_w"))
            .set("dh", ctx->getAttrUInt("dilate_h"))
            .set("dw", ctx->getAttrUInt("dilate_w"));
    return s.text;
}

// Workspace: the space-to-depth tensor of the first-layer form, nothing otherwise. The
// reference sizes workspaces by running this function at compile time (JIT); the CUDA
// pack also answers directly through WorkspaceBytes().
std::string ConvBiasQS8::GetWorkspaceBody(TContext* ctx) const {
    Subst s{R"(
TinyNNStatus ${signature} {
    mb200_conv_param p;
    ${symbol}_param(inputs, &p);
    *workspace = mb200_conv_s2d_supported(&p) ? mb200_conv_s2d_workspace_bytes(&p) : 0;
    return TinyNN_SUCCESS;
}
)"};
    s.set("signature", GetWorkspaceSignature(ctx)).set("symbol", GetKernelSymbol(ctx));
    return s.text;
}

size_t ConvBiasQS8::WorkspaceBytes(TContext* ctx) const {
    const CCOperand src = ctx->getAttrOprand("operand:0");
    const CCOperand flt = ctx->getAttrOprand("operand:1");
    const CCOperand dst = last_operand(ctx);
    const int form = filter_form(ctx);
    if (form < 0 || (form == 0 && (src.shape.size() != 4 || dst.shape.size() != 4)))
        return 0;
    auto channels = [](const CCOperand& o) {
        return (int)(o.shape.size() == 5 ? o.shape[1] * 4 : o.shape[1]);
    };
    const int groups = ctx->getAttrStr("sparse") == "DENSE" ? 1
                                                            : (int)flt.shape[0] * (form ? 4 : 1);
    const mb200::S2dGeom g = mb200::s2d_geometry(
            (int)src.shape[0], channels(src), (int)src.shape[2], (int)src.shape[3],
            channels(dst), (int)ctx->getAttrUInt("kernel_h"), (int)ctx->getAttrUInt("kernel_w"),
            (int)ctx->getAttrUInt("stride_h"), (int)ctx->getAttrUInt("stride_w"),
            (int)ctx->getAttrUInt("pad_h"), (int)ctx->getAttrUInt("pad_w"),
            (int)ctx->getAttrUInt("dilate_h"), (int)ctx->getAttrUInt("dilate_w"), groups);
    return g.ok ? g.workspace_bytes : 0;
}

// ------------------------------------------------------------------------------------------
// Pooling
// ------------------------------------------------------------------------------------------
bool PoolingQS8::IsAvailable(TContext* ctx) const {
    if (ctx->getAttrStr("format") != "NCHW")
        return false;
    const CCOperand src = ctx->getAttrOprand("operand:0");
    const CCOperand dst = ctx->getAttrOprand("operand:1");
    if (!is_quant(src.dtype, 8) || !is_quant(dst.dtype, 8))
        return false;
    // quantised pooling keeps the scale (compiler/lib/KernelGen/BareMetal/Pooling.cpp:22-27)
    if (src.scale != dst.scale)
        return false;
    const std::string mode = ctx->getAttrStr("mode");
    return mode == "MAX" || mode == "AVERAGE" || mode == "AVERAGE_COUNT_EXCLUDE_PADDING";
}

std::string PoolingQS8::GetKernelSymbol(TContext* ctx) const {
    std::stringstream ss;
    ss << "cuda_sm100_pooling_" << ctx->getAttrStr("mode") << "_NHWC_p" << ctx->getAttrInt("pad_h")
       << "x" << ctx->getAttrInt("pad_w") << "_s" << ctx->getAttrInt("stride_h") << "x"
       << ctx->getAttrInt("stride_w") << "_w" << ctx->getAttrInt("window_h") << "x"
       << ctx->getAttrInt("window_w") << "_" << io_str(ctx);
    return ss.str();
}

std::string PoolingQS8::GetKernelBody(TContext* ctx) const {
    const std::string mode = ctx->getAttrStr("mode");
    Subst s{R"(
${prologue}
TinyNNStatus ${signature} {
    const Tensor* src = inputs[0];
    return (TinyNNStatus)mb200_pooling_qs8_nhwc(
            (const int8_t*)src->ptr, (int8_t*)outputs[0]->ptr, ${mode}, src->layout.dims[0],
            src->layout.dims[1], src->layout.dims[2], src->layout.dims[3], ${wh}, ${ww}, ${sh},
            ${sw}, ${ph}, ${pw}, mb200_opt_stream(opt));
}
)"};
    s.set("prologue", GenStubPrologue())
            .set("signature", GetKernelSignature(ctx))
            .set("mode", mode == "MAX" ? 0 : mode == "AVERAGE" ? 1 : 2)
            .set("wh", ctx->getAttrInt("window_h"))
            .set("ww", ctx->getAttrInt("window_w"))
            .set("sh", ctx->getAttrInt("stride_h"))
            .set("sw", ctx->getAttrInt("stride_w"))
            .set("ph", ctx->getAttrInt("pad_h"))
            .set("pw", ctx->getAttrInt("pad_w"));
    return s.text;
}

// ------------------------------------------------------------------------------------------
// ElemwiseMultiType
// ------------------------------------------------------------------------------------------
static int qelem_code(const std::string& m) {
    return m == "QADD" ? 0 : m == "QFUSE_ADD_RELU" ? 1 : m == "QMUL" ? 2 : m == "QRELU" ? 3 : -1;
}

bool ElemwiseMultiTypeQS8::IsAvailable(TContext* ctx) const {
    const std::string mode = ctx->getAttrStr("mode");
    const int n = ctx->getAttrInt("nr_operands");
    if (qelem_code(mode) < 0)
        return false;
    if ((mode == "QRELU") != (n == 2) || (n != 2 && n != 3))
        return false;
    for (int i = 0; i < n; ++i)
        if (!is_quant(ctx->getAttrOprand("operand:" + std::to_string(i)).dtype, 8))
            return false;
    // same-shape operands only; the broadcast forms stay on the reference's CPU kernels
    if (n == 3 && ctx->getAttrOprand("operand:0").shape != ctx->getAttrOprand("operand:1").shape)
        return false;
    return true;
}

std::string ElemwiseMultiTypeQS8::GetKernelSymbol(TContext* ctx) const {
    return "cuda_sm100_elementwise_multitype_" + ctx->getAttrStr("mode") + "_" + io_str(ctx);
}

std::string ElemwiseMultiTypeQS8::GetKernelBody(TContext* ctx) const {
    const bool unary = ctx->getAttrInt("nr_operands") == 2;
    Subst s{R"(
${prologue}
TinyNNStatus ${signature} {
    const Tensor* a = inputs[0];
    const Tensor* b = ${unary} ? inputs[0] : inputs[1];
    size_t nr_elem = 1;
    for (int i = 0; i < a->layout.nr_dim; ++i) nr_elem *= a->layout.dims[i];
    return (TinyNNStatus)mb200_qelemwise_qs8(
            (const int8_t*)a->ptr, (const int8_t*)b->ptr, (int8_t*)outputs[0]->ptr, ${mode},
            nr_elem, a->dtype.param.scale, b->dtype.param.scale, outputs[0]->dtype.param.scale,
            mb200_opt_stream(opt));
}
)"};
    s.set("prologue", GenStubPrologue())
            .set("signature", GetKernelSignature(ctx))
            .set("unary", unary ? 1 : 0)
            .set("mode", qelem_code(ctx->getAttrStr("mode")));
    return s.text;
}

// ------------------------------------------------------------------------------------------
// TypeCvt
// ------------------------------------------------------------------------------------------
bool TypeCvtQS32QS8::IsAvailable(TContext* ctx) const {
    const CCOperand src = ctx->getAttrOprand("operand:0");
    const CCOperand dst = ctx->getAttrOprand("operand:1");
    return is_quant(src.dtype, 32) && is_quant(dst.dtype, 8) && src.scale > 0 && dst.scale > 0;
}

std::string TypeCvtQS32QS8::GetKernelSymbol(TContext* ctx) const {
    return "cuda_sm100_typecvt_" + io_str(ctx);
}

std::string TypeCvtQS32QS8::GetKernelBody(TContext* ctx) const {
    Subst s{R"(
${prologue}
TinyNNStatus ${signature} {
    const Tensor* src = inputs[0];
    size_t nr_elem = 1;
    for (int i = 0; i < src->layout.nr_dim; ++i) nr_elem *= src->layout.dims[i];
    return (TinyNNStatus)mb200_typecvt_qs32_qs8(
            (const int32_t*)src->ptr, (int8_t*)outputs[0]->ptr, nr_elem, src->dtype.param.scale,
            outputs[0]->dtype.param.scale, mb200_opt_stream(opt));
}
)"};
    s.set("prologue", GenStubPrologue()).set("signature", GetKernelSignature(ctx));
    return s.text;
}

// ------------------------------------------------------------------------------------------
// MatrixMul (+ TypeCvt)
// ------------------------------------------------------------------------------------------
bool MatMulQS8::IsAvailable(TContext* ctx) const {
    if (!ctx->haveAttr("fused_typecvt") || ctx->getAttrStr("format") != "DEFAULT" ||
        ctx->getAttrStr("compute_mode") != "DEFAULT")
        return false;
    if (ctx->getAttrBool("transposeA") || ctx->getAttrBool("transposeB"))
        return false;
    const CCOperand a = ctx->getAttrOprand("operand:0");
    const CCOperand b = ctx->getAttrOprand("operand:1");
    const CCOperand c = ctx->getAttrOprand("operand:2");
    return is_quant(a.dtype, 8) && is_quant(b.dtype, 8) && is_quant(c.dtype, 8) && a.scale > 0 &&
           b.scale > 0 && c.scale > 0;
}

std::string MatMulQS8::GetKernelSymbol(TContext*) const {
    // kernel_matmul_<n|t><n|t>_<dtype> in the reference; the requantisation is spelled out
    return "cuda_sm100_matmul_nn_qsi8qsi8qsi32_typecvt_qsi8";
}

std::string MatMulQS8::GetKernelBody(TContext* ctx) const {
    Subst s{R"(
${prologue}
TinyNNStatus ${signature} {
    const Tensor* a = inputs[0];
    const Tensor* b = inputs[1]; /* re-laid to [N][K] by the init function */
    Tensor* c = outputs[0];
    const int m = a->layout.dims[0];
    int k = 1;
    for (int i = 1; i < a->layout.nr_dim; ++i) k *= a->layout.dims[i];
    const int n = c->layout.dims[1];
    /* scale of the qint32 product as MegEngine records it: one float multiplication */
    const float acc_scale = a->dtype.param.scale * b->dtype.param.scale;
    return (TinyNNStatus)mb200_matmul_s8_qs8(
            m, n, k, (const int8_t*)a->ptr, (const int8_t*)b->ptr, (int8_t*)c->ptr, acc_scale,
            c->dtype.param.scale, mb200_opt_stream(opt));
}
)"};
    s.set("prologue", GenStubPrologue()).set("signature", GetKernelSignature(ctx));
    return s.text;
}

std::string MatMulQS8::GetInitBody(TContext* ctx) const {
    Subst s{R"(
${prologue}
TinyNNStatus ${signature} {
    /* three-phase init (runtime/src/data_struct.h:135-142): B [K][N] -> [N][K] on the device */
    Tensor* b = inputs[1];
    const int k = b->layout.dims[0], n = b->layout.dims[1];
    if (out_weights == NULL && nr_out_weight != NULL) {
        *nr_out_weight = 1;
        return TinyNN_SUCCESS;
    }
    if (out_weights != NULL && nr_out_weight == NULL) {
        out_weights[0].layout.nr_dim = 2;
        out_weights[0].layout.dims[0] = n;
        out_weights[0].layout.dims[1] = k;
        out_weights[0].layout.stride[0] = k;
        out_weights[0].layout.stride[1] = 1;
        out_weights[0].dtype = b->dtype;
        out_weights[0].name = b->name;
        return TinyNN_SUCCESS;
    }
    return (TinyNNStatus)mb200_matmul_pack_b(
            k, n, (const int8_t*)b->ptr, (int8_t*)out_weights[0].ptr, mb200_opt_stream(opt));
}
)"};
    s.set("prologue", GenStubPrologue()).set("signature", GetInitSignature(ctx));
    return s.text;
}

// ------------------------------------------------------------------------------------------
// Relayout
// ------------------------------------------------------------------------------------------
bool RelayoutQS8::IsAvailable(TContext* ctx) const {
    if (!ctx->haveAttr("relayout_mode"))
        return false;
    const std::string m = ctx->getAttrStr("relayout_mode");
    const CCOperand src = ctx->getAttrOprand("operand:0");
    if (m == "NCHW44_NHWC")  // [N][C/4][H][W][4] in
        return src.shape.size() == 5 && src.shape[4] == 4 && is_quant(src.dtype, 8);
    if (m == "NHWC_NCHW44")
        return src.shape.size() == 4 && src.shape[1] % 4 == 0 && is_quant(src.dtype, 8);
    return (m == "NCHW_NHWC" || m == "NHWC_NCHW") && src.shape.size() == 4 &&
           (is_quant(src.dtype, 8) || src.dtype == "si8" || src.dtype == "f32");
}

std::string RelayoutQS8::GetKernelSymbol(TContext* ctx) const {
    return "cuda_sm100_relayout_" + ctx->getAttrStr("relayout_mode") + "_" + io_str(ctx);
}

std::string RelayoutQS8::GetKernelBody(TContext* ctx) const {
    const std::string m = ctx->getAttrStr("relayout_mode");
    if (m == "NCHW44_NHWC" || m == "NHWC_NCHW44") {
        Subst s{R"(
${prologue}
TinyNNStatus ${signature} {
    const Tensor* src = inputs[0];
    return (TinyNNStatus)${fn}(
            (const int8_t*)src->ptr, (int8_t*)outputs[0]->ptr, src->layout.dims[0],
            src->layout.dims[1] * ${cblock}, src->layout.dims[2], src->layout.dims[3],
            mb200_opt_stream(opt));
}
)"};
        const bool from44 = m == "NCHW44_NHWC";
        s.set("prologue", GenStubPrologue())
                .set("signature", GetKernelSignature(ctx))
                .set("cblock", from44 ? 4 : 1)
                .set("fn", from44 ? "mb200_relayout_nchw44_to_nhwc_s8"
                                  : "mb200_relayout_nhwc_to_nchw44_s8");
        return s.text;
    }
    const bool to_nhwc = m == "NCHW_NHWC";
    Subst s{R"(
${prologue}
TinyNNStatus ${signature} {
    const Tensor* src = inputs[0];
    return (TinyNNStatus)${fn}(
            (const ${ctype}*)src->ptr, (${ctype}*)outputs[0]->ptr, src->layout.dims[0],
            src->layout.dims[1], src->layout.dims[2], src->layout.dims[3], mb200_opt_stream(opt));
}
)"};
    const bool f32 = ctx->getAttrOprand("operand:0").dtype == "f32";
    s.set("prologue", GenStubPrologue())
            .set("signature", GetKernelSignature(ctx))
            .set("ctype", f32 ? "float" : "int8_t")
            .set("fn", std::string(to_nhwc ? "mb200_relayout_nchw_to_nhwc_" : "mb200_relayout_nhwc_to_nchw_") +
                               (f32 ? "f32" : "s8"));
    return s.text;
}

// ==========================================================================================
// fp32 path
// ==========================================================================================
namespace {

bool all_f32(TContext* ctx) {
    const int n = ctx->getAttrInt("nr_operands");
    for (int i = 0; i < n; ++i) {
        const CCOperand o = ctx->getAttrOprand("operand:" + std::to_string(i));
        // an absent bias is an operand without a shape (Common/ConvKernel.h:10-21)
        if (o.dtype != "f32" && !(o.shape.empty() && i == 2))
            return false;
    }
    return true;
}

int f32_act_code(const std::string& m) {
    return m == "RELU" ? 1 : m == "H_SWISH" ? 2 : m == "SIGMOID" ? 3 : m == "SILU" ? 4 : 0;
}

int elem_code(const std::string& m) {
    static const char* names[] = {"RELU", "SIGMOID", "SILU", "H_SWISH", "EXP"};
    for (int i = 0; i < 5; ++i)
        if (m == names[i])
            return i;
    static const char* bin[] = {"ADD", "SUB", "MUL", "MAX", "FUSE_ADD_RELU"};
    for (int i = 0; i < 5; ++i)
        if (m == bin[i])
            return 16 + i;
    return -1;
}

// the C text that fills an mb200_conv_f32_param from the Tensors of a ConvBias
const char* kConvF32ParamFn = R"(
static void ${symbol}_param(Tensor** inputs, mb200_conv_f32_param* p) {
    const Tensor* src = inputs[0];
    p->n = src->layout.dims[0];
    p->ic = src->layout.dims[1];
    p->ih = src->layout.dims[2];
    p->iw = src->layout.dims[3];
    p->groups = ${dense} ? 1 : p->ic / ${icpg};
    p->oc = ${oc};
    p->kh = ${kh}; p->kw = ${kw};
    p->stride_h = ${sh}; p->stride_w = ${sw};
    p->pad_h = ${ph}; p->pad_w = ${pw};
    p->nonline = ${nonline};
}
)";

Subst conv_f32_common(TContext* ctx, const KernelFunc* self, const char* text) {
    Subst s{text};
    const CCOperand dst = last_operand(ctx);
    s.set("prologue", GenStubPrologue())
            .set("symbol", self->GetKernelSymbol(ctx))
            .set("oc", (long long)dst.shape[1])
            .set("kh", ctx->getAttrUInt("kernel_h"))
            .set("kw", ctx->getAttrUInt("kernel_w"))
            .set("sh", ctx->getAttrUInt("stride_h"))
            .set("sw", ctx->getAttrUInt("stride_w"))
            .set("ph", ctx->getAttrUInt("pad_h"))
            .set("pw", ctx->getAttrUInt("pad_w"))
            .set("dense", ctx->getAttrStr("sparse") == "DENSE" ? 1 : 0)
            .set("icpg", ctx->getAttrStr("sparse") == "DENSE"
                                 ? 1LL
                                 : (long long)ctx->getAttrOprand("operand:1").shape[2])
            .set("nonline", f32_act_code(nonline(ctx)));
    return s;
}

}  // namespace

bool ConvBiasF32::IsAvailable(TContext* ctx) const {
    if (ctx->getAttrStr("format") != "NCHW" || ctx->getAttrStr("mode") != "CROSS_CORRELATION")
        return false;
    const int n = ctx->getAttrInt("nr_operands");
    if (n < 4 || n > 5 || !all_f32(ctx))
        return false;
    if (ctx->getAttrUInt("dilate_h") != 1 || ctx->getAttrUInt("dilate_w") != 1)
        return false;
    const CCOperand src = ctx->getAttrOprand("operand:0");
    const CCOperand dst = last_operand(ctx);
    if (src.shape.size() != 4 || dst.shape.size() != 4)
        return false;
    const std::string sparse = ctx->getAttrStr("sparse");
    if (sparse != "DENSE" && sparse != "GROUP")
        return false;
    const std::string act = nonline(ctx);
    if (act != "IDENTITY" && act != "RELU" && act != "SIGMOID" && act != "H_SWISH" &&
        act != "SILU")
        return false;
    if (has_bias(ctx) && !channel_broadcast_bias(ctx))
        return false;
    const std::string fm = fuse_mode(ctx);
    if (n == 5) {
        if (fm != "ADD" || ctx->getAttrOprand("operand:3").shape != dst.shape)
            return false;
    } else if (!fm.empty()) {
        return false;
    }
    return true;
}

std::string ConvBiasF32::GetKernelSymbol(TContext* ctx) const {
    if (!ctx)
        return "cuda_sm100_conv2d_f32";
    std::stringstream ss;
    ss << "cuda_sm100_conv2d_" << ctx->getAttrUInt("kernel_h") << "x"
       << ctx->getAttrUInt("kernel_w") << "_NHWC_" << ctx->getAttrStr("sparse") << "_p"
       << ctx->getAttrUInt("pad_h") << "x" << ctx->getAttrUInt("pad_w") << "_s"
       << ctx->getAttrUInt("stride_h") << "x" << ctx->getAttrUInt("stride_w") << "_d1x1_oc"
       << last_operand(ctx).shape[1];
    // the processed filter is a flat buffer, so a grouped filter's channels per group are
    // spelled out ([G][OCpg][ICpg][KH][KW])
    if (ctx->getAttrStr("sparse") == "GROUP")
        ss << "_icpg" << ctx->getAttrOprand("operand:1").shape[2];
    ss << "_f32";
    if (has_bias(ctx))
        ss << "_bias";
    if (nonline(ctx) != "IDENTITY")
        ss << "_" << nonline(ctx);
    if (!fuse_mode(ctx).empty())
        ss << "_z_" << fuse_mode(ctx);
    return ss.str();
}

std::string ConvBiasF32::GetKernelBody(TContext* ctx) const {
    std::string text = std::string("${prologue}") + kConvF32ParamFn + R"(
/* dims are the logical NCHW extents; strides say the buffers are NHWC. The pixel pitch of
 * the output (stride of W) may exceed its channel count: the output is then a channel slice
 * of a wider buffer, which is how a Concat of ConvBias results needs no copy. */
TinyNNStatus ${signature} {
    const Tensor* src = inputs[0];
    Tensor* dst = outputs[0];
    mb200_conv_f32_param p;
    ${symbol}_param(inputs, &p);
    const float* bias = ${has_bias} ? (const float*)inputs[2]->ptr : 0;
    const float* z = ${fused} ? (const float*)inputs[nr_input - 1]->ptr : 0;
    return (TinyNNStatus)mb200_conv_bias_f32_nhwc(
            &p, (const float*)src->ptr, (const float*)inputs[1]->ptr, bias, z, (float*)dst->ptr,
            (long long)dst->layout.stride[3], workspace->ptr, workspace->size, MB200_ALGO_AUTO,
            mb200_opt_stream(opt));
}
)";
    Subst s = conv_f32_common(ctx, this, text.c_str());
    s.set("signature", GetKernelSignature(ctx))
            .set("has_bias", has_bias(ctx) ? 1 : 0)
            .set("fused", fuse_mode(ctx).empty() ? 0 : 1);
    return s.text;
}

std::string ConvBiasF32::GetInitBody(TContext* ctx) const {
    Subst s = conv_f32_common(ctx, this, R"(
TinyNNStatus ${signature} {
    /* three-phase init (runtime/src/data_struct.h:135-142): the OIHW filter becomes the K-major
     * filter followed by its two tf32 planes, a flat float buffer */
    Tensor* in_weights = inputs[1];
    mb200_conv_f32_param p;
    ${symbol}_param(inputs, &p);
    if (out_weights == 0 && nr_out_weight != 0) {
        *nr_out_weight = 1;
        return TinyNN_SUCCESS;
    }
    if (out_weights != 0 && nr_out_weight == 0) {
        out_weights->layout.nr_dim = 1;
        out_weights->layout.dims[0] = (uint32_t)(mb200_conv_f32_packed_filter_bytes(&p) / 4);
        out_weights->layout.stride[0] = 1;
        out_weights->layout.format = in_weights->layout.format;
        out_weights->dtype = in_weights->dtype;
        out_weights->name = in_weights->name;
        return TinyNN_SUCCESS;
    }
    return (TinyNNStatus)mb200_conv_f32_pack_filter(
            &p, (const float*)in_weights->ptr, (float*)out_weights->ptr, mb200_opt_stream(opt));
}
)");
    s.set("signature", GetInitSignature(ctx));
    return s.text;
}

std::string ConvBiasF32::GetWorkspaceBody(TContext* ctx) const {
    Subst s = conv_f32_common(ctx, this, R"(
TinyNNStatus ${signature} {
    mb200_conv_f32_param p;
    ${symbol}_param(inputs, &p);
    *workspace = mb200_conv_f32_workspace_bytes(&p);
    return TinyNN_SUCCESS;
}
)");
    s.set("signature", GetWorkspaceSignature(ctx));
    return s.text;
}

// must agree with mb200_conv_f32_workspace_bytes (megcc_b200/csrc/f32_abi.cu): the two tf32
// planes of the activation when the filter is dense and its channels fill whole TMA rows
size_t ConvBiasF32::WorkspaceBytes(TContext*) const {
    return 0;  // the activation is split into its tf32 planes in shared memory
}

// ---- MatrixMul fp32 ----
bool MatMulF32::IsAvailable(TContext* ctx) const {
    if (ctx->haveAttr("fused_typecvt") || ctx->getAttrStr("format") != "DEFAULT")
        return false;
    if (ctx->getAttrBool("transposeA") || ctx->getAttrBool("transposeB"))
        return false;
    return ctx->getAttrInt("nr_operands") == 3 && all_f32(ctx);
}

std::string MatMulF32::GetKernelSymbol(TContext*) const {
    return "cuda_sm100_matmul_nn_f32f32f32";
}

std::string MatMulF32::GetKernelBody(TContext* ctx) const {
    Subst s{R"(
${prologue}
TinyNNStatus ${signature} {
    const Tensor* a = inputs[0];
    const Tensor* b = inputs[1]; /* prepared by the init function */
    Tensor* c = outputs[0];
    const int m = a->layout.dims[0];
    int k = 1;
    for (int i = 1; i < a->layout.nr_dim; ++i) k *= a->layout.dims[i];
    const int n = c->layout.dims[1];
    return (TinyNNStatus)mb200_matmul_f32(
            m, n, k, (const float*)a->ptr, (const float*)b->ptr, (float*)c->ptr, workspace->ptr,
            workspace->size, mb200_opt_stream(opt));
}
)"};
    s.set("prologue", GenStubPrologue()).set("signature", GetKernelSignature(ctx));
    return s.text;
}

std::string MatMulF32::GetInitBody(TContext* ctx) const {
    Subst s{R"(
${prologue}
TinyNNStatus ${signature} {
    Tensor* b = inputs[1];
    const int k = b->layout.dims[0], n = b->layout.dims[1];
    if (out_weights == NULL && nr_out_weight != NULL) {
        *nr_out_weight = 1;
        return TinyNN_SUCCESS;
    }
    if (out_weights != NULL && nr_out_weight == NULL) {
        out_weights[0].layout.nr_dim = 1;
        out_weights[0].layout.dims[0] = (uint32_t)(mb200_matmul_f32_packed_b_bytes(k, n) / 4);
        out_weights[0].layout.stride[0] = 1;
        out_weights[0].dtype = b->dtype;
        out_weights[0].name = b->name;
        return TinyNN_SUCCESS;
    }
    return (TinyNNStatus)mb200_matmul_f32_pack_b(
            k, n, (const float*)b->ptr, (float*)out_weights[0].ptr, mb200_opt_stream(opt));
}
)"};
    s.set("prologue", GenStubPrologue()).set("signature", GetInitSignature(ctx));
    return s.text;
}

std::string MatMulF32::GetWorkspaceBody(TContext* ctx) const {
    Subst s{R"(
TinyNNStatus ${signature} {
    const Tensor* a = inputs[0];
    int k = 1;
    for (int i = 1; i < a->layout.nr_dim; ++i) k *= a->layout.dims[i];
    *workspace = mb200_matmul_f32_workspace_bytes((int)a->layout.dims[0], k);
    return TinyNN_SUCCESS;
}
)"};
    s.set("signature", GetWorkspaceSignature(ctx));
    return s.text;
}

size_t MatMulF32::WorkspaceBytes(TContext*) const {
    return 0;
}

// ---- Elemwise fp32 ----
bool ElemwiseF32::IsAvailable(TContext* ctx) const {
    const int code = elem_code(ctx->getAttrStr("mode"));
    const int n = ctx->getAttrInt("nr_operands");
    if (code < 0 || !all_f32(ctx))
        return false;
    if ((code < 16) != (n == 2) || (n != 2 && n != 3))
        return false;
    // same-shape operands only
    return n == 2 || ctx->getAttrOprand("operand:0").shape == ctx->getAttrOprand("operand:1").shape;
}

std::string ElemwiseF32::GetKernelSymbol(TContext* ctx) const {
    return "cuda_sm100_elementwise_" + ctx->getAttrStr("mode") + "_" + io_str(ctx);
}

std::string ElemwiseF32::GetKernelBody(TContext* ctx) const {
    Subst s{R"(
${prologue}
TinyNNStatus ${signature} {
    const Tensor* a = inputs[0];
    const Tensor* b = nr_input > 1 ? inputs[1] : inputs[0];
    size_t nr_elem = 1;
    for (int i = 0; i < a->layout.nr_dim; ++i) nr_elem *= a->layout.dims[i];
    return (TinyNNStatus)mb200_elemwise_f32(
            ${mode}, (const float*)a->ptr, (const float*)b->ptr, (float*)outputs[0]->ptr, nr_elem,
            mb200_opt_stream(opt));
}
)"};
    s.set("prologue", GenStubPrologue())
            .set("signature", GetKernelSignature(ctx))
            .set("mode", elem_code(ctx->getAttrStr("mode")));
    return s.text;
}

// ---- Concat / Focus ----
bool ConcatF32::IsAvailable(TContext* ctx) const {
    if (ctx->getAttrInt("axis") != 1 || !all_f32(ctx))
        return false;
    const int n = ctx->getAttrInt("nr_operands");
    if (ctx->haveAttr("focus"))
        return n == 2 && ctx->getAttrOprand("operand:0").shape.size() == 4;
    return n >= 2 && n <= 9;
}

std::string ConcatF32::GetKernelSymbol(TContext* ctx) const {
    if (ctx->haveAttr("focus"))
        return "cuda_sm100_concat_focus_f32";
    return "cuda_sm100_concat_NHWC_axis_1_f32";
}

std::string ConcatF32::GetKernelBody(TContext* ctx) const {
    if (ctx->haveAttr("focus")) {
        Subst s{R"(
${prologue}
/* the four stride-2 slices of the NCHW input, concatenated along channels, as NHWC */
TinyNNStatus ${signature} {
    const Tensor* src = inputs[0];
    return (TinyNNStatus)mb200_focus_f32(
            (const float*)src->ptr, (float*)outputs[0]->ptr, src->layout.dims[0],
            src->layout.dims[1], src->layout.dims[2], src->layout.dims[3],
            outputs[0]->layout.dims[1], mb200_opt_stream(opt));
}
)"};
        s.set("prologue", GenStubPrologue()).set("signature", GetKernelSignature(ctx));
        return s.text;
    }
    Subst s{R"(
${prologue}
TinyNNStatus ${signature} {
    const float* srcs[8];
    int channels[8];
    if (nr_input > 8) return TinyNN_ERROR_OUT_OF_RANGE;
    for (int i = 0; i < nr_input; ++i) {
        srcs[i] = (const float*)inputs[i]->ptr;
        channels[i] = inputs[i]->layout.dims[1];
    }
    const Tensor* dst = outputs[0];
    return (TinyNNStatus)mb200_concat_f32_nhwc(
            srcs, channels, nr_input, (float*)dst->ptr,
            (size_t)dst->layout.dims[0] * dst->layout.dims[2] * dst->layout.dims[3],
            mb200_opt_stream(opt));
}
)"};
    s.set("prologue", GenStubPrologue()).set("signature", GetKernelSignature(ctx));
    return s.text;
}

// ---- Resize ----
bool ResizeF32::IsAvailable(TContext* ctx) const {
    return ctx->getAttrStr("imode") == "NEAREST" && ctx->getAttrStr("format") == "NCHW" &&
           ctx->getAttrOprand("operand:0").dtype == "f32" &&
           ctx->getAttrOprand("operand:0").shape.size() == 4;
}

std::string ResizeF32::GetKernelSymbol(TContext*) const {
    return "cuda_sm100_resize_NHWC_NEAREST_f32";
}

std::string ResizeF32::GetKernelBody(TContext* ctx) const {
    Subst s{R"(
${prologue}
TinyNNStatus ${signature} {
    const Tensor* src = inputs[0];
    const Tensor* dst = outputs[0];
    return (TinyNNStatus)mb200_resize_nearest_f32_nhwc(
            (const float*)src->ptr, (float*)dst->ptr, src->layout.dims[0], src->layout.dims[1],
            src->layout.dims[2], src->layout.dims[3], dst->layout.dims[2], dst->layout.dims[3],
            mb200_opt_stream(opt));
}
)"};
    s.set("prologue", GenStubPrologue()).set("signature", GetKernelSignature(ctx));
    return s.text;
}

// ---- Pooling fp32 ----
bool PoolingF32::IsAvailable(TContext* ctx) const {
    if (ctx->getAttrStr("format") != "NCHW" || !all_f32(ctx))
        return false;
    const std::string mode = ctx->getAttrStr("mode");
    return mode == "MAX" || mode == "AVERAGE" || mode == "AVERAGE_COUNT_EXCLUDE_PADDING";
}

std::string PoolingF32::GetKernelSymbol(TContext* ctx) const {
    std::stringstream ss;
    ss << "cuda_sm100_pooling_" << ctx->getAttrStr("mode") << "_NHWC_p" << ctx->getAttrInt("pad_h")
       << "x" << ctx->getAttrInt("pad_w") << "_s" << ctx->getAttrInt("stride_h") << "x"
       << ctx->getAttrInt("stride_w") << "_w" << ctx->getAttrInt("window_h") << "x"
       << ctx->getAttrInt("window_w") << "_" << io_str(ctx);
    return ss.str();
}

std::string PoolingF32::GetKernelBody(TContext* ctx) const {
    const std::string mode = ctx->getAttrStr("mode");
    Subst s{R"(
${prologue}
TinyNNStatus ${signature} {
    const Tensor* src = inputs[0];
    return (TinyNNStatus)mb200_pooling_f32_nhwc(
            (const float*)src->ptr, (float*)outputs[0]->ptr, ${mode}, src->layout.dims[0],
            src->layout.dims[1], src->layout.dims[2], src->layout.dims[3], ${wh}, ${ww}, ${sh},
            ${sw}, ${ph}, ${pw}, mb200_opt_stream(opt));
}
)"};
    s.set("prologue", GenStubPrologue())
            .set("signature", GetKernelSignature(ctx))
            .set("mode", mode == "MAX" ? 0 : mode == "AVERAGE" ? 1 : 2)
            .set("wh", ctx->getAttrInt("window_h"))
            .set("ww", ctx->getAttrInt("window_w"))
            .set("sh", ctx->getAttrInt("stride_h"))
            .set("sw", ctx->getAttrInt("stride_w"))
            .set("ph", ctx->getAttrInt("pad_h"))
            .set("pw", ctx->getAttrInt("pad_w"));
    return s.text;
}

// ------------------------------------------------------------------------------------------
std::vector<const KernelFunc*> ArchKernelPack::GetKernel(KernelPack::KernType kernel_type) {
    static ConvBiasQS8 conv;
    static PoolingQS8 pooling;
    static ElemwiseMultiTypeQS8 qelem;
    static TypeCvtQS32QS8 typecvt;
    static RelayoutQS8 relayout;
    static MatMulQS8 matmul;
    static ConvBiasF32 conv_f32;
    static MatMulF32 matmul_f32;
    static ElemwiseF32 elem_f32;
    static ConcatF32 concat_f32;
    static ResizeF32 resize_f32;
    static PoolingF32 pooling_f32;
    switch (kernel_type) {
        case KernelPack::KernType::MatrixMulKernel:
            return {&matmul, &matmul_f32};
        case KernelPack::KernType::ConvKernel:
            return {&conv, &conv_f32};
        case KernelPack::KernType::PoolingKernel:
            return {&pooling, &pooling_f32};
        case KernelPack::KernType::ElemwiseKernel:
            return {&elem_f32};
        case KernelPack::KernType::ConcatKernel:
            return {&concat_f32};
        case KernelPack::KernType::ResizeKernel:
            return {&resize_f32};
        case KernelPack::KernType::ElemwiseMultiKernel:
            return {&qelem};
        case KernelPack::KernType::TypeCvtKernel:
            return {&typecvt};
        case KernelPack::KernType::RelayoutKernel:
            return {&relayout};
        default:
            return {};
    }
}
