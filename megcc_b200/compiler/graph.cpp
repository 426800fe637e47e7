// Network description -> kernel selection -> static memory plan -> tinynn model.
// See include/megcc_b200_compiler.h for what each step replaces in the reference.
#include <stdarg.h>
#include <string.h>

#include <algorithm>
#include <fstream>
#include <map>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/megcc_b200_compiler.h"
#include "../csrc/tinynn_format.h"
#include "cuda_kernel_pack.h"

namespace fb = tinynn_fb;
using namespace megcc;
using KernType = KernelGen::KernelPack::KernType;

namespace {

thread_local char g_err[512] = "";
int err(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return -1;
}

struct GTensor {
    std::string name;
    int c = 0, h = 0, w = 0;  // per image
    float scale = 1.f;
    bool nchw = false;  // physical layout of the buffer (model input / 1x1 outputs)
    bool is_input = false, is_output = false;
    bool f32 = false;   // fp32 tensor (else qint8)
    // model-visible tensor of an NCHW44 model: buffer [N][C/4][H][W][4]
    bool nchw44 = false;
};

struct GWeight {
    std::string name;
    fb::DTypeEnum dtype;
    float scale;
    std::vector<int> dims;
    std::vector<uint8_t> data;
    int use_count = 0;
};

enum class OpType { CONV, POOL, QELEM, RELAYOUT, MATMUL, ELEM_F32, CONCAT, FOCUS, RESIZE };

struct GOp {
    OpType type;
    std::string name;
    std::vector<int> inputs;   // tensor ids
    std::vector<int> weights;  // weight ids, appended after the tensor inputs
    int output = -1;
    // conv / pooling
    int kh = 0, kw = 0, stride = 1, pad = 0, groups = 1;
    std::string mode;  // nonline / pooling mode / elemwise mode / relayout mode
    bool has_bias = false;
    float flt_scale = 1.f;
    // a fused ElemwiseMultiType step behind a ConvBias: inputs = {src, z}
    std::string fuse_mode;  // "" | "QADD" | "QFUSE_ADD_RELU"
    float mid_scale = 1.f;  // scale of the ConvBias result that the fused step consumes
    int mid_weight = -1;    // 1-element float weight carrying mid_scale to the runtime
    bool f32 = false;       // fp32 operator (CONV / MATMUL / POOL / RELAYOUT)
    // ConvBias whose filter is given in an NCHW44 layout: 1 dense, 2 channel-wise, 3 first
    // layer (NCHW input)
    int flt44 = 0;
    // ConvBias with the MAX pooling 3x3 / stride 2 / pad 1 behind it folded in: output is
    // the pooled tensor
    bool pool_fused = false;
};

struct Compiled {
    size_t arena = 0, unplanned = 0;
};

std::string qdtype(const char* base, float scale) {
    uint32_t bits;
    memcpy(&bits, &scale, 4);
    std::stringstream ss;
    ss << base << "<" << bits << ":" << scale << ">";
    return ss.str();
}

CCOperand operand(const char* base, std::vector<size_t> shape, float scale) {
    CCOperand o;
    o.shape = std::move(shape);
    o.dtype = qdtype(base, scale);
    o.scale = scale;
    return o;
}

CCOperand operand_f32(std::vector<size_t> shape) {
    CCOperand o;
    o.shape = std::move(shape);
    o.dtype = "f32";
    o.scale = 1.f;
    return o;
}

#ifdef MEGCC_B200_IN_MEGCC_TREE
void set_u32(CodeGenContext& c, const char* k, uint32_t v) { c.setAttr(k, CCAttr(v)); }
void set_i32(CodeGenContext& c, const char* k, int32_t v) { c.setAttr(k, CCAttr(v)); }
void set_str(CodeGenContext& c, const char* k, const std::string& v) { c.setAttr(k, CCAttr(v)); }
void set_opr(CodeGenContext& c, const std::string& k, const CCOperand& v) { c.setAttr(k, CCAttr(v)); }
void set_bool(CodeGenContext& c, const char* k, bool v) { c.setAttr(k, CCAttr(v)); }
#else
void set_u32(CodeGenContext& c, const char* k, uint32_t v) { c.setInt(k, v); }
void set_i32(CodeGenContext& c, const char* k, int32_t v) { c.setInt(k, v); }
void set_str(CodeGenContext& c, const char* k, const std::string& v) { c.setStr(k, v); }
void set_opr(CodeGenContext& c, const std::string& k, const CCOperand& v) { c.setOperand(k, v); }
void set_bool(CodeGenContext& c, const char* k, bool v) { c.setInt(k, v ? 1 : 0); }
#endif

int out_extent(int in, int k, int s, int p) {
    return (in + 2 * p - (k - 1) - 1) / s + 1;
}

}  // namespace

struct mb200c_graph {
    std::string name;
    std::vector<GTensor> tensors;
    std::vector<GWeight> weights;
    std::vector<GOp> ops;
    // results of the last compile
    std::vector<uint8_t> bytes;
    std::vector<std::string> symbols;
    std::map<std::string, const KernelGen::KernelFunc*> kernel_of;
    std::map<std::string, std::shared_ptr<CodeGenContext>> ctx_of;
    std::string symbols_joined;
    std::vector<Compiled> compiled;
    bool fuse_conv_elemwise = true;
    // ConvBias + MAX pooling as one instruction: off unless asked for (on a ResNet-18 stem
    // at batch 256 the fused kernel measured 217 us against 132 + 55 us for the pair)
    bool fuse_conv_pooling = false;
    // 0: CUDA_SM100 DeviceModels only; 1: a BARE_METAL DeviceModel per batch beside them
    // (the operators as the reference's own x86 kernels: one artefact for both runtimes);
    // 2: the BARE_METAL DeviceModels alone
    int bare_metal_model = 0;

    int add_tensor(const std::string& n, int c, int h, int w, float scale) {
        GTensor t;
        t.name = n;
        t.c = c;
        t.h = h;
        t.w = w;
        t.scale = scale;
        tensors.push_back(t);
        return (int)tensors.size() - 1;
    }
    bool valid(int id) const { return id >= 0 && (size_t)id < tensors.size(); }

    // the attribute bag KernelMaterialization would build for this operator and batch
    // (KernelMaterialization.cpp:136-158; attribute names of MGBToKernelHelper.h:98-124)
    std::shared_ptr<CodeGenContext> context_for(const GOp& op, int batch) const {
        auto ctx = std::make_shared<CodeGenContext>();
        auto shape = [&](int id) {
            const GTensor& t = tensors[id];
            return std::vector<size_t>{(size_t)batch, (size_t)t.c, (size_t)t.h, (size_t)t.w};
        };
        auto topr = [&](int id) {
            const GTensor& t = tensors[id];
            return t.f32 ? operand_f32(shape(id)) : operand("qsi8", shape(id), t.scale);
        };
        switch (op.type) {
            case OpType::ELEM_F32: {
                set_str(*ctx, "mode", op.mode);
                int k = 0;
                for (int id : op.inputs)
                    set_opr(*ctx, "operand:" + std::to_string(k++), topr(id));
                set_opr(*ctx, "operand:" + std::to_string(k++), topr(op.output));
                set_i32(*ctx, "nr_operands", k);
                break;
            }
            case OpType::CONCAT:
            case OpType::FOCUS: {
                set_i32(*ctx, "axis", 1);
                if (op.type == OpType::FOCUS)
                    set_i32(*ctx, "focus", 1);
                int k = 0;
                for (int id : op.inputs)
                    set_opr(*ctx, "operand:" + std::to_string(k++), topr(id));
                set_opr(*ctx, "operand:" + std::to_string(k++), topr(op.output));
                set_i32(*ctx, "nr_operands", k);
                break;
            }
            case OpType::RESIZE: {
                set_str(*ctx, "imode", "NEAREST");
                set_str(*ctx, "format", "NCHW");
                set_opr(*ctx, "operand:0", topr(op.inputs[0]));
                set_opr(*ctx, "operand:1", topr(op.output));
                set_i32(*ctx, "nr_operands", 2);
                break;
            }
            case OpType::CONV: {
                const GTensor& src = tensors[op.inputs[0]];
                const GTensor& dst = tensors[op.output];
                set_u32(*ctx, "kernel_h", op.kh);
                set_u32(*ctx, "kernel_w", op.kw);
                set_u32(*ctx, "stride_h", op.stride);
                set_u32(*ctx, "stride_w", op.stride);
                set_u32(*ctx, "pad_h", op.pad);
                set_u32(*ctx, "pad_w", op.pad);
                set_u32(*ctx, "dilate_h", 1);
                set_u32(*ctx, "dilate_w", 1);
                set_str(*ctx, "sparse", op.groups == 1 ? "DENSE" : "GROUP");
                set_str(*ctx, "format", op.flt44 ? "NCHW44" : "NCHW");
                set_str(*ctx, "mode", "CROSS_CORRELATION");
                set_str(*ctx, "nonlineMode", op.mode);
                set_str(*ctx, "compute_mode", "DEFAULT");
                if (op.pool_fused)
                    set_str(*ctx, "fuse_pooling", "MAX_3x3_s2x2_p1x1");
                if (op.f32) {
                    std::vector<size_t> fshape;
                    for (int d : weights[op.weights[0]].dims)
                        fshape.push_back(d);
                    set_opr(*ctx, "operand:0", topr(op.inputs[0]));
                    set_opr(*ctx, "operand:1", operand_f32(fshape));
                    set_opr(*ctx, "operand:2", op.has_bias ? operand_f32({1, (size_t)dst.c, 1, 1})
                                                           : operand_f32({}));
                    if (op.inputs.size() > 1) {
                        set_opr(*ctx, "operand:3", topr(op.inputs[1]));
                        set_opr(*ctx, "operand:4", topr(op.output));
                        set_i32(*ctx, "nr_operands", 5);
                        set_str(*ctx, "fuse_elemwise_mode", "ADD");
                    } else {
                        set_opr(*ctx, "operand:3", topr(op.output));
                        set_i32(*ctx, "nr_operands", 4);
                    }
                    break;
                }
                // what the operator looks like in an NCHW44 graph: 5-dim tensors, except the
                // NCHW input of the first layer
                auto shape_of = [&](int id, bool blocked) {
                    const GTensor& t = tensors[id];
                    if (!blocked)
                        return shape(id);
                    return std::vector<size_t>{(size_t)batch, (size_t)t.c / 4, (size_t)t.h,
                                               (size_t)t.w, 4};
                };
                const bool b_src = op.flt44 == 1 || op.flt44 == 2, b_dst = op.flt44 != 0;
                set_opr(*ctx, "operand:0",
                        operand("qsi8", shape_of(op.inputs[0], b_src), src.scale));
                std::vector<size_t> fs;
                for (int d : weights[op.weights[0]].dims)
                    fs.push_back(d);
                set_opr(*ctx, "operand:1", operand("qsi8", fs, op.flt_scale));
                if (op.has_bias && b_dst)
                    set_opr(*ctx, "operand:2",
                            operand("qsi32", {1, (size_t)dst.c / 4, 1, 1, 4},
                                    src.scale * op.flt_scale));
                else if (op.has_bias)
                    set_opr(*ctx, "operand:2",
                            operand("qsi32", {1, (size_t)dst.c, 1, 1}, src.scale * op.flt_scale));
                else
                    set_opr(*ctx, "operand:2", operand("qsi32", {}, src.scale * op.flt_scale));
                if (op.fuse_mode.empty()) {
                    set_opr(*ctx, "operand:3",
                            operand("qsi8", shape_of(op.output, b_dst), dst.scale));
                    set_i32(*ctx, "nr_operands", 4);
                } else {
                    // operand order src, filter, bias, z, dst: the z slot of the reference's
                    // Conv2DKernel (include/compiler/Dialect/Kernel/IR/AbstractKernels.td:113-118)
                    set_opr(*ctx, "operand:3",
                            operand("qsi8", shape_of(op.inputs[1], b_dst),
                                    tensors[op.inputs[1]].scale));
                    set_opr(*ctx, "operand:4",
                            operand("qsi8", shape_of(op.output, b_dst), dst.scale));
                    set_i32(*ctx, "nr_operands", 5);
                    set_str(*ctx, "fuse_elemwise_mode", op.fuse_mode);
#ifdef MEGCC_B200_IN_MEGCC_TREE
                    ctx->setAttr("fuse_mid_scale", CCAttr(op.mid_scale));
#else
                    ctx->setFloat("fuse_mid_scale", op.mid_scale);
#endif
                }
                break;
            }
            case OpType::POOL: {
                set_str(*ctx, "mode", op.mode);
                set_str(*ctx, "format", "NCHW");
                set_i32(*ctx, "window_h", op.kh);
                set_i32(*ctx, "window_w", op.kw);
                set_i32(*ctx, "stride_h", op.stride);
                set_i32(*ctx, "stride_w", op.stride);
                set_i32(*ctx, "pad_h", op.pad);
                set_i32(*ctx, "pad_w", op.pad);
                set_opr(*ctx, "operand:0", topr(op.inputs[0]));
                set_opr(*ctx, "operand:1", topr(op.output));
                set_i32(*ctx, "nr_operands", 2);
                break;
            }
            case OpType::QELEM: {
                set_str(*ctx, "mode", op.mode);
                int k = 0;
                for (int id : op.inputs)
                    set_opr(*ctx, "operand:" + std::to_string(k++),
                            operand("qsi8", shape(id), tensors[id].scale));
                set_opr(*ctx, "operand:" + std::to_string(k++),
                        operand("qsi8", shape(op.output), tensors[op.output].scale));
                set_i32(*ctx, "nr_operands", k);
                break;
            }
            case OpType::MATMUL: {
                // MatrixMul qsi8 x qsi8 -> qsi32 with the TypeCvt behind it folded in
                // (attribute names of BareMetal/MatrixMul.cpp:13-43)
                const GTensor& a = tensors[op.inputs[0]];
                const GTensor& c = tensors[op.output];
                const GWeight& b = weights[op.weights[0]];
                set_bool(*ctx, "transposeA", false);
                set_bool(*ctx, "transposeB", false);
                set_str(*ctx, "format", "DEFAULT");
                set_str(*ctx, "compute_mode", "DEFAULT");
                if (op.f32) {
                    set_opr(*ctx, "operand:0",
                            operand_f32({(size_t)batch, (size_t)(a.c * a.h * a.w)}));
                    set_opr(*ctx, "operand:1",
                            operand_f32({(size_t)b.dims[0], (size_t)b.dims[1]}));
                    set_opr(*ctx, "operand:2", operand_f32({(size_t)batch, (size_t)c.c}));
                    set_i32(*ctx, "nr_operands", 3);
                    break;
                }
                set_str(*ctx, "fused_typecvt", "qsi8");
                set_opr(*ctx, "operand:0",
                        operand("qsi8", {(size_t)batch, (size_t)(a.c * a.h * a.w)}, a.scale));
                set_opr(*ctx, "operand:1",
                        operand("qsi8", {(size_t)b.dims[0], (size_t)b.dims[1]}, b.scale));
                set_opr(*ctx, "operand:2", operand("qsi8", {(size_t)batch, (size_t)c.c}, c.scale));
                set_i32(*ctx, "nr_operands", 3);
                break;
            }
            case OpType::RELAYOUT: {
                set_str(*ctx, "relayout_mode", op.mode);
                auto side = [&](int id) {
                    const GTensor& t = tensors[id];
                    if (!t.nchw44)
                        return topr(id);
                    return operand("qsi8",
                                   {(size_t)batch, (size_t)t.c / 4, (size_t)t.h, (size_t)t.w, 4},
                                   t.scale);
                };
                set_opr(*ctx, "operand:0", side(op.inputs[0]));
                set_opr(*ctx, "operand:1", side(op.output));
                set_i32(*ctx, "nr_operands", 2);
                break;
            }
        }
        return ctx;
    }

    static KernType kern_type(OpType t) {
        switch (t) {
            case OpType::CONV: return KernType::ConvKernel;
            case OpType::POOL: return KernType::PoolingKernel;
            case OpType::QELEM: return KernType::ElemwiseMultiKernel;
            case OpType::MATMUL: return KernType::MatrixMulKernel;
            case OpType::ELEM_F32: return KernType::ElemwiseKernel;
            case OpType::CONCAT:
            case OpType::FOCUS: return KernType::ConcatKernel;
            case OpType::RESIZE: return KernType::ResizeKernel;
            default: return KernType::RelayoutKernel;
        }
    }
};

namespace {

size_t tensor_bytes(const GTensor& t, int batch) {
    return (size_t)batch * t.c * t.h * t.w * (t.f32 ? 4 : 1);
}

size_t align256(size_t v) {
    return (v + 255) / 256 * 256;
}

// Static memory planning: every tensor lives from the instruction that writes it to the
// last one that reads it (inputs from the start, outputs to the end); tensors are placed
// largest first at the lowest 256-byte aligned offset that is free for their whole
// lifetime. Returns the arena size.
size_t plan_memory(
        const mb200c_graph& g, const std::vector<GOp>& ops, int batch,
        const std::vector<size_t>& ws_bytes, std::vector<size_t>* offsets,
        std::vector<size_t>* ws_offsets, size_t* unplanned) {
    const size_t n = g.tensors.size();
    std::vector<int> first(n, -1), last(n, -1);
    for (size_t i = 0; i < n; ++i)
        if (g.tensors[i].is_input)
            first[i] = 0;
    for (size_t k = 0; k < ops.size(); ++k) {
        for (int id : ops[k].inputs) {
            if (first[id] < 0)
                first[id] = (int)k;
            last[id] = (int)k;
        }
        if (first[ops[k].output] < 0)
            first[ops[k].output] = (int)k;
        last[ops[k].output] = std::max(last[ops[k].output], (int)k);
    }
    for (size_t i = 0; i < n; ++i)
        if (g.tensors[i].is_output)
            last[i] = (int)ops.size();
    std::vector<size_t> order;
    for (size_t i = 0; i < n; ++i)
        if (first[i] >= 0)
            order.push_back(i);
    std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) {
        return tensor_bytes(g.tensors[a], batch) > tensor_bytes(g.tensors[b], batch);
    });
    // workspaces are planned as extra buffers that live for exactly one instruction
    struct Item {
        size_t bytes;
        int first, last;
        size_t offset;
    };
    std::vector<Item> items;
    for (size_t i = 0; i < n; ++i)
        items.push_back({first[i] >= 0 ? align256(tensor_bytes(g.tensors[i], batch)) : 0, first[i],
                         last[i], 0});
    for (size_t k = 0; k < ops.size(); ++k)
        items.push_back({align256(ws_bytes[k]), ws_bytes[k] ? (int)k : -1, (int)k, 0});
    order.clear();
    for (size_t i = 0; i < items.size(); ++i)
        if (items[i].first >= 0 && items[i].bytes)
            order.push_back(i);
    std::stable_sort(order.begin(), order.end(),
                     [&](size_t a, size_t b) { return items[a].bytes > items[b].bytes; });
    std::vector<size_t> placed;
    size_t arena = 0;
    *unplanned = 0;
    for (size_t id : order) {
        const size_t sz = items[id].bytes;
        *unplanned += sz;
        // gather busy intervals of buffers alive at the same time
        std::vector<std::pair<size_t, size_t>> busy;
        for (size_t o : placed)
            if (!(items[o].last < items[id].first || items[id].last < items[o].first))
                busy.push_back({items[o].offset, items[o].offset + items[o].bytes});
        std::sort(busy.begin(), busy.end());
        size_t off = 0;
        for (auto& b : busy) {
            if (off + sz <= b.first)
                break;
            off = std::max(off, b.second);
        }
        items[id].offset = off;
        arena = std::max(arena, off + sz);
        placed.push_back(id);
    }
    offsets->assign(n, 0);
    for (size_t i = 0; i < n; ++i)
        (*offsets)[i] = items[i].offset;
    ws_offsets->assign(ops.size(), 0);
    for (size_t k = 0; k < ops.size(); ++k)
        (*ws_offsets)[k] = items[n + k].offset;
    return arena;
}

fb::NodeP dtype_node(fb::DTypeEnum t, float scale) {
    auto p = fb::make_table();
    p->add<float>(fb::field::DP_scale, scale);
    auto d = fb::make_table();
    d->add<int8_t>(fb::field::DT_type, (int8_t)t);
    d->add_ref(fb::field::DT_param, p);
    return d;
}

fb::NodeP layout_node(const std::vector<int>& dims, const std::vector<int>& stride, fb::Format f) {
    auto l = fb::make_table();
    l->add_ref(fb::field::L_dims, fb::make_vec<int32_t>(dims));
    l->add_ref(fb::field::L_stride, fb::make_vec<int32_t>(stride));
    l->add<int8_t>(fb::field::L_format, (int8_t)f);
    return l;
}

std::vector<int> contiguous(const std::vector<int>& dims) {
    std::vector<int> s(dims.size(), 1);
    for (int i = (int)dims.size() - 2; i >= 0; --i)
        s[i] = s[i + 1] * dims[i + 1];
    return s;
}

}  // namespace

// ---------------------------------------------------------------------------------------
extern "C" {

const char* mb200c_last_error(void) {
    return g_err;
}

mb200c_graph* mb200c_graph_create(const char* model_name) {
    auto* g = new mb200c_graph();
    g->name = model_name ? model_name : "model";
    return g;
}

void mb200c_graph_destroy(mb200c_graph* g) {
    delete g;
}

int mb200c_add_input(mb200c_graph* g, const char* name, int c, int h, int w, float scale) {
    if (!g || !name || c <= 0 || h <= 0 || w <= 0 || !(scale > 0))
        return err("add_input: bad argument");
    const int id = g->add_tensor(name, c, h, w, scale);
    g->tensors[id].is_input = true;
    g->tensors[id].nchw = true;
    return id;
}

int mb200c_add_input_nchw44(mb200c_graph* g, const char* name, int c, int h, int w, float scale) {
    if (!g || !name || c <= 0 || c % 4 || h <= 0 || w <= 0 || !(scale > 0))
        return err("add_input_nchw44: bad argument (channels must be a multiple of 4)");
    const int id = g->add_tensor(name, c, h, w, scale);
    g->tensors[id].is_input = true;
    g->tensors[id].nchw44 = true;
    return id;
}

int mb200c_add_conv_bias_nchw44(
        mb200c_graph* g, const char* name, int src, int oc, int kh, int kw, int stride, int pad,
        int groups, const char* nonline, const int8_t* flt44, float flt_scale,
        const int32_t* bias, const float* channel_scales, float dst_scale) {
    if (!g || !g->valid(src) || !name)
        return err("add_conv_bias_nchw44: bad argument");
    const GTensor s = g->tensors[src];
    int form;
    if (groups == 1 && s.is_input && s.nchw && !s.nchw44)
        form = 3;  // NCHW model input -> NCHW44
    else if (groups == 1)
        form = 1;
    else if (groups == s.c && oc == s.c)
        form = 2;
    else
        return err("add_conv_bias_nchw44 %s: only dense and channel-wise filters have an NCHW44 "
                   "layout here", name);
    if (oc % 4 || (form != 3 && s.c % 4))
        return err("add_conv_bias_nchw44 %s: channels must be multiples of 4", name);
    // same operator; the filter bytes are taken as they are (the count is the same)
    const int out = mb200c_add_conv_bias(g, name, src, oc, kh, kw, stride, pad, groups, nonline,
                                         flt44, flt_scale, bias, channel_scales, dst_scale);
    if (out < 0)
        return out;
    GOp& op = g->ops.back();
    op.flt44 = form;
    GWeight& wf = g->weights[op.weights[0]];
    if (form == 1)
        wf.dims = {oc / 4, s.c / 4, kh, kw, 4, 4};
    else if (form == 2)
        wf.dims = {oc / 4, 1, 1, kh, kw, 4};
    else
        wf.dims = {oc / 4, kh, kw, s.c, 4};
    if (op.has_bias)
        g->weights[op.weights[1]].dims = {1, oc / 4, 1, 1, 4};
    return out;
}

int mb200c_add_conv_bias(
        mb200c_graph* g, const char* name, int src, int oc, int kh, int kw, int stride, int pad,
        int groups, const char* nonline, const int8_t* flt, float flt_scale, const int32_t* bias,
        const float* channel_scales, float dst_scale) {
    if (!g || !name || !nonline || !flt || !g->valid(src) || g->tensors[src].f32)
        return err("add_conv_bias: bad argument");
    const GTensor s = g->tensors[src];
    if (oc <= 0 || kh <= 0 || kw <= 0 || stride <= 0 || pad < 0 || groups <= 0 ||
        s.c % groups || oc % groups)
        return err("add_conv_bias %s: bad extents", name);
    const int oh = out_extent(s.h, kh, stride, pad), ow = out_extent(s.w, kw, stride, pad);
    if (oh <= 0 || ow <= 0)
        return err("add_conv_bias %s: filter larger than padded input", name);
    GOp op;
    op.type = OpType::CONV;
    op.name = name;
    op.inputs = {src};
    op.kh = kh;
    op.kw = kw;
    op.stride = stride;
    op.pad = pad;
    op.groups = groups;
    op.mode = nonline;
    op.flt_scale = flt_scale;
    const int icpg = s.c / groups;
    GWeight wf;
    wf.name = std::string(name) + ":filter";
    wf.dtype = fb::QInt8;
    wf.scale = flt_scale;
    wf.dims = groups == 1 ? std::vector<int>{oc, s.c, kh, kw}
                          : std::vector<int>{groups, oc / groups, icpg, kh, kw};
    wf.data.assign((const uint8_t*)flt, (const uint8_t*)flt + (size_t)oc * icpg * kh * kw);
    wf.use_count = 1;
    g->weights.push_back(std::move(wf));
    op.weights.push_back((int)g->weights.size() - 1);
    if (bias) {
        GWeight wb;
        wb.name = std::string(name) + ":bias";
        wb.dtype = fb::QInt32;
        wb.scale = s.scale * flt_scale;
        wb.dims = {1, oc, 1, 1};
        wb.data.assign((const uint8_t*)bias, (const uint8_t*)bias + (size_t)oc * 4);
        wb.use_count = 1;
        g->weights.push_back(std::move(wb));
        op.weights.push_back((int)g->weights.size() - 1);
        op.has_bias = true;
    }
    if (channel_scales) {
        GWeight ws;
        ws.name = std::string(name) + ":channel_scales";
        ws.dtype = fb::Float32;
        ws.scale = 1.f;
        ws.dims = {oc};
        ws.data.assign((const uint8_t*)channel_scales, (const uint8_t*)channel_scales + (size_t)oc * 4);
        ws.use_count = 1;
        g->weights.push_back(std::move(ws));
        op.weights.push_back((int)g->weights.size() - 1);
    }
    op.output = g->add_tensor(std::string(name) + ":out", oc, oh, ow, dst_scale);
    g->ops.push_back(op);
    return op.output;
}

int mb200c_add_matmul(
        mb200c_graph* g, const char* name, int src, int n, const int8_t* b, float b_scale,
        float dst_scale) {
    if (!g || !name || !b || !g->valid(src) || n <= 0)
        return err("add_matmul: bad argument");
    const GTensor s = g->tensors[src];
    const int k = s.c * s.h * s.w;
    if (s.h != 1 || s.w != 1)
        return err("add_matmul %s: the input must be a [batch][K] matrix (h = w = 1)", name);
    GOp op;
    op.type = OpType::MATMUL;
    op.name = name;
    op.inputs = {src};
    op.flt_scale = b_scale;
    GWeight wb;
    wb.name = std::string(name) + ":B";
    wb.dtype = fb::QInt8;
    wb.scale = b_scale;
    wb.dims = {k, n};
    wb.data.assign((const uint8_t*)b, (const uint8_t*)b + (size_t)k * n);
    wb.use_count = 1;
    g->weights.push_back(std::move(wb));
    op.weights.push_back((int)g->weights.size() - 1);
    op.output = g->add_tensor(std::string(name) + ":out", n, 1, 1, dst_scale);
    g->ops.push_back(op);
    return op.output;
}

int mb200c_add_input_f32(mb200c_graph* g, const char* name, int c, int h, int w) {
    const int id = mb200c_add_input(g, name, c, h, w, 1.f);
    if (id >= 0)
        g->tensors[id].f32 = true;
    return id;
}

int mb200c_add_conv_f32(
        mb200c_graph* g, const char* name, int src, int oc, int kh, int kw, int stride, int pad,
        int groups, const char* nonline, const float* flt, const float* bias, int z) {
    if (!g || !name || !nonline || !flt || !g->valid(src) || !g->tensors[src].f32)
        return err("add_conv_f32: bad argument");
    const GTensor s = g->tensors[src];
    if (oc <= 0 || kh <= 0 || kw <= 0 || stride <= 0 || pad < 0 || groups <= 0 ||
        s.c % groups || oc % groups)
        return err("add_conv_f32 %s: bad extents", name);
    const int oh = out_extent(s.h, kh, stride, pad), ow = out_extent(s.w, kw, stride, pad);
    if (oh <= 0 || ow <= 0)
        return err("add_conv_f32 %s: filter larger than padded input", name);
    if (z >= 0) {
        if (!g->valid(z) || !g->tensors[z].f32 || g->tensors[z].c != oc ||
            g->tensors[z].h != oh || g->tensors[z].w != ow)
            return err("add_conv_f32 %s: z does not have the output's shape", name);
    }
    GOp op;
    op.type = OpType::CONV;
    op.f32 = true;
    op.name = name;
    op.inputs = z >= 0 ? std::vector<int>{src, z} : std::vector<int>{src};
    op.kh = kh;
    op.kw = kw;
    op.stride = stride;
    op.pad = pad;
    op.groups = groups;
    op.mode = nonline;
    const int icpg = s.c / groups;
    GWeight wf;
    wf.name = std::string(name) + ":filter";
    wf.dtype = fb::Float32;
    wf.scale = 1.f;
    wf.dims = groups == 1 ? std::vector<int>{oc, s.c, kh, kw}
                          : std::vector<int>{groups, oc / groups, icpg, kh, kw};
    wf.data.assign((const uint8_t*)flt, (const uint8_t*)flt + (size_t)oc * icpg * kh * kw * 4);
    wf.use_count = 1;
    g->weights.push_back(std::move(wf));
    op.weights.push_back((int)g->weights.size() - 1);
    if (bias) {
        GWeight wb;
        wb.name = std::string(name) + ":bias";
        wb.dtype = fb::Float32;
        wb.scale = 1.f;
        wb.dims = {1, oc, 1, 1};
        wb.data.assign((const uint8_t*)bias, (const uint8_t*)bias + (size_t)oc * 4);
        wb.use_count = 1;
        g->weights.push_back(std::move(wb));
        op.weights.push_back((int)g->weights.size() - 1);
        op.has_bias = true;
    }
    op.output = g->add_tensor(std::string(name) + ":out", oc, oh, ow, 1.f);
    g->tensors[op.output].f32 = true;
    g->ops.push_back(op);
    return op.output;
}

int mb200c_add_matmul_f32(mb200c_graph* g, const char* name, int src, int n, const float* b) {
    if (!g || !name || !b || !g->valid(src) || n <= 0 || !g->tensors[src].f32)
        return err("add_matmul_f32: bad argument");
    const GTensor s = g->tensors[src];
    if (s.h != 1 || s.w != 1)
        return err("add_matmul_f32 %s: the input must be a [batch][K] matrix (h = w = 1)", name);
    GOp op;
    op.type = OpType::MATMUL;
    op.f32 = true;
    op.name = name;
    op.inputs = {src};
    GWeight wb;
    wb.name = std::string(name) + ":B";
    wb.dtype = fb::Float32;
    wb.scale = 1.f;
    wb.dims = {s.c, n};
    wb.data.assign((const uint8_t*)b, (const uint8_t*)b + (size_t)s.c * n * 4);
    wb.use_count = 1;
    g->weights.push_back(std::move(wb));
    op.weights.push_back((int)g->weights.size() - 1);
    op.output = g->add_tensor(std::string(name) + ":out", n, 1, 1, 1.f);
    g->tensors[op.output].f32 = true;
    g->ops.push_back(op);
    return op.output;
}

int mb200c_add_elemwise_f32(mb200c_graph* g, const char* name, const char* mode, int a, int b) {
    if (!g || !name || !mode || !g->valid(a) || !g->tensors[a].f32)
        return err("add_elemwise_f32: bad argument");
    const GTensor s = g->tensors[a];
    GOp op;
    op.type = OpType::ELEM_F32;
    op.f32 = true;
    op.name = name;
    op.mode = mode;
    op.inputs = {a};
    if (b >= 0) {
        if (!g->valid(b) || !g->tensors[b].f32 || g->tensors[b].c != s.c ||
            g->tensors[b].h != s.h || g->tensors[b].w != s.w)
            return err("add_elemwise_f32 %s: operand shapes differ", name);
        op.inputs.push_back(b);
    }
    op.output = g->add_tensor(std::string(name) + ":out", s.c, s.h, s.w, 1.f);
    g->tensors[op.output].f32 = true;
    g->ops.push_back(op);
    return op.output;
}

int mb200c_add_concat(mb200c_graph* g, const char* name, const int* srcs, int nr) {
    if (!g || !name || !srcs || nr < 1 || nr > 8)
        return err("add_concat: 1..8 inputs");
    GOp op;
    op.type = OpType::CONCAT;
    op.f32 = true;
    op.name = name;
    int c = 0;
    for (int i = 0; i < nr; ++i) {
        if (!g->valid(srcs[i]) || !g->tensors[srcs[i]].f32)
            return err("add_concat %s: input %d is not an fp32 tensor", name, i);
        const GTensor& t = g->tensors[srcs[i]];
        if (t.h != g->tensors[srcs[0]].h || t.w != g->tensors[srcs[0]].w)
            return err("add_concat %s: spatial extents differ", name);
        c += t.c;
        op.inputs.push_back(srcs[i]);
    }
    const GTensor s = g->tensors[srcs[0]];
    op.output = g->add_tensor(std::string(name) + ":out", c, s.h, s.w, 1.f);
    g->tensors[op.output].f32 = true;
    g->ops.push_back(op);
    return op.output;
}

int mb200c_add_focus(mb200c_graph* g, const char* name, int src, int c_out) {
    if (!g || !name || !g->valid(src) || !g->tensors[src].f32)
        return err("add_focus: bad argument");
    const GTensor s = g->tensors[src];
    if (!s.nchw || (s.h & 1) || (s.w & 1) || c_out < 4 * s.c)
        return err("add_focus %s: needs the NCHW model input with even extents and "
                   "c_out >= 4 * c", name);
    GOp op;
    op.type = OpType::FOCUS;
    op.f32 = true;
    op.name = name;
    op.inputs = {src};
    op.output = g->add_tensor(std::string(name) + ":out", c_out, s.h / 2, s.w / 2, 1.f);
    g->tensors[op.output].f32 = true;
    g->ops.push_back(op);
    return op.output;
}

int mb200c_add_resize_nearest(mb200c_graph* g, const char* name, int src, int oh, int ow) {
    if (!g || !name || !g->valid(src) || !g->tensors[src].f32 || oh <= 0 || ow <= 0)
        return err("add_resize_nearest: bad argument");
    const GTensor s = g->tensors[src];
    GOp op;
    op.type = OpType::RESIZE;
    op.f32 = true;
    op.name = name;
    op.inputs = {src};
    op.output = g->add_tensor(std::string(name) + ":out", s.c, oh, ow, 1.f);
    g->tensors[op.output].f32 = true;
    g->ops.push_back(op);
    return op.output;
}

int mb200c_add_pooling(
        mb200c_graph* g, const char* name, int src, const char* mode, int window, int stride,
        int pad) {
    if (!g || !name || !mode || !g->valid(src) || window <= 0 || stride <= 0 || pad < 0)
        return err("add_pooling: bad argument");
    const GTensor s = g->tensors[src];
    const int oh = (s.h + 2 * pad - window) / stride + 1, ow = (s.w + 2 * pad - window) / stride + 1;
    if (s.h + 2 * pad < window || s.w + 2 * pad < window)
        return err("add_pooling %s: window larger than padded input", name);
    GOp op;
    op.type = OpType::POOL;
    op.name = name;
    op.inputs = {src};
    op.kh = op.kw = window;
    op.stride = stride;
    op.pad = pad;
    op.mode = mode;
    op.f32 = s.f32;
    op.output = g->add_tensor(std::string(name) + ":out", s.c, oh, ow, s.scale);
    g->tensors[op.output].f32 = s.f32;
    g->ops.push_back(op);
    return op.output;
}

int mb200c_add_qelemwise(
        mb200c_graph* g, const char* name, const char* mode, int a, int b, float dst_scale) {
    if (!g || !name || !mode || !g->valid(a))
        return err("add_qelemwise: bad argument");
    if (g->tensors[a].f32)
        return err("add_qelemwise %s: fp32 tensors take add_elemwise_f32", name);
    const bool unary = strcmp(mode, "QRELU") == 0;
    if (!unary && !g->valid(b))
        return err("add_qelemwise %s: second operand missing", name);
    const GTensor s = g->tensors[a];
    if (!unary) {
        const GTensor& t = g->tensors[b];
        if (t.c != s.c || t.h != s.h || t.w != s.w)
            return err("add_qelemwise %s: operand shapes differ", name);
    }
    GOp op;
    op.type = OpType::QELEM;
    op.name = name;
    op.inputs = unary ? std::vector<int>{a} : std::vector<int>{a, b};
    op.mode = mode;
    op.output = g->add_tensor(std::string(name) + ":out", s.c, s.h, s.w, dst_scale);
    g->ops.push_back(op);
    return op.output;
}

int mb200c_set_option(mb200c_graph* g, const char* name, int value) {
    if (!g || !name)
        return err("set_option: bad argument");
    if (strcmp(name, "bare_metal_model") == 0) {
        if (value < 0 || value > 2)
            return err("set_option: bare_metal_model is 0, 1 or 2");
        g->bare_metal_model = value;
        return 0;
    }
    if (strcmp(name, "fuse_conv_pooling") == 0) {
        g->fuse_conv_pooling = value != 0;
        return 0;
    }
    if (strcmp(name, "fuse_conv_elemwise") == 0) {
        g->fuse_conv_elemwise = value != 0;
        return 0;
    }
    return err("set_option: unknown option '%s'", name);
}

int mb200c_mark_output(mb200c_graph* g, int tensor) {
    if (!g || !g->valid(tensor))
        return err("mark_output: bad tensor id");
    g->tensors[tensor].is_output = true;
    return 0;
}

int mb200c_compile(
        mb200c_graph* g, const int* batches, int nr_batches, const uint8_t** bytes, size_t* len) {
    if (!g || !batches || nr_batches <= 0 || !bytes || !len)
        return err("compile: bad argument");
    g->symbols.clear();
    g->kernel_of.clear();
    g->ctx_of.clear();
    g->compiled.clear();

    // ---- layout decisions: activations are NHWC inside the model; the model input is
    // NCHW (read in place by a first ConvBias, else converted); outputs are handed back
    // in NCHW, which is free for 1x1 maps and costs a Relayout otherwise ----
    mb200c_graph work = *g;  // ops get relayouts inserted; the user's graph stays as is
    {
        std::vector<GOp> ops;
        std::map<int, int> nhwc_of;  // NCHW input id -> converted tensor id
        // a model with NCHW44 inputs or filters hands its outputs back in NCHW44 too
        bool model44 = false;
        for (auto& t : work.tensors)
            model44 |= t.nchw44;
        for (auto& op : work.ops)
            model44 |= op.flt44 != 0;
        for (auto op : work.ops) {
            for (size_t k = 0; k < op.inputs.size(); ++k) {
                const int id = op.inputs[k];
                if (work.tensors[id].nchw44 && !nhwc_of.count(id)) {
                    const GTensor t = work.tensors[id];
                    const int nid = work.add_tensor(t.name + ":nhwc", t.c, t.h, t.w, t.scale);
                    GOp r;
                    r.type = OpType::RELAYOUT;
                    r.name = t.name + ":to_nhwc";
                    r.inputs = {id};
                    r.mode = "NCHW44_NHWC";
                    r.output = nid;
                    ops.push_back(r);
                    nhwc_of[id] = nid;
                }
                if (work.tensors[id].nchw44) {
                    op.inputs[k] = nhwc_of[id];
                    continue;
                }
                if (!work.tensors[id].nchw)
                    continue;
                if ((op.type == OpType::CONV && !op.f32 && k == 0) || op.type == OpType::FOCUS)
                    continue;  // the qint8 ConvBias and Focus read NCHW directly
                if (work.tensors[id].h == 1 && work.tensors[id].w == 1)
                    continue;  // NCHW == NHWC
                if (!nhwc_of.count(id)) {
                    const GTensor t = work.tensors[id];
                    const int nid = work.add_tensor(t.name + ":nhwc", t.c, t.h, t.w, t.scale);
                    work.tensors[nid].f32 = t.f32;
                    GOp r;
                    r.f32 = t.f32;
                    r.type = OpType::RELAYOUT;
                    r.name = t.name + ":to_nhwc";
                    r.inputs = {id};
                    r.mode = "NCHW_NHWC";
                    r.output = nid;
                    ops.push_back(r);
                    nhwc_of[id] = nid;
                }
                op.inputs[k] = nhwc_of[id];
            }
            ops.push_back(op);
        }
        const size_t n_before = work.tensors.size();
        for (size_t id = 0; id < n_before; ++id) {
            GTensor& t = work.tensors[id];
            if (!t.is_output || t.nchw || t.nchw44)
                continue;
            const bool to44 = model44 && !t.f32 && t.c % 4 == 0;
            if (t.h == 1 && t.w == 1 && !to44) {  // one pixel: NCHW is the channel vector
                t.nchw = true;
                continue;
            }
            if (to44) {
                // (also for a single pixel: the visible tensor has five dims, the operator
                // that produces it works on four)
                const GTensor copy = t;
                t.is_output = false;
                const int nid = work.add_tensor(copy.name + ":nchw44", copy.c, copy.h, copy.w,
                                                copy.scale);
                work.tensors[nid].is_output = true;
                work.tensors[nid].nchw44 = true;
                std::swap(work.tensors[id].name, work.tensors[nid].name);
                GOp r;
                r.type = OpType::RELAYOUT;
                r.name = copy.name + ":to_nchw44";
                r.inputs = {(int)id};
                r.mode = "NHWC_NCHW44";
                r.output = nid;
                ops.push_back(r);
                continue;
            }
            const GTensor copy = t;
            t.is_output = false;
            const int nid = work.add_tensor(copy.name + ":nchw", copy.c, copy.h, copy.w, copy.scale);
            work.tensors[nid].is_output = true;
            work.tensors[nid].nchw = true;
            work.tensors[nid].f32 = copy.f32;
            std::swap(work.tensors[id].name, work.tensors[nid].name);  // keep the visible name
            GOp r;
            r.f32 = copy.f32;
            r.type = OpType::RELAYOUT;
            r.name = copy.name + ":to_nchw";
            r.inputs = {(int)id};
            r.mode = "NHWC_NCHW";
            r.output = nid;
            ops.push_back(r);
        }
        work.ops = ops;
    }

    // ---- fusion: ConvBias (no activation) whose only consumer is a QADD / QFUSE_ADD_RELU
    // becomes one instruction at the consumer's position; the other operand is z ----
    if (g->fuse_conv_elemwise) {
        std::vector<int> uses(work.tensors.size(), 0), producer(work.tensors.size(), -1);
        for (size_t k = 0; k < work.ops.size(); ++k) {
            for (int id : work.ops[k].inputs)
                uses[id]++;
            producer[work.ops[k].output] = (int)k;
        }
        std::vector<char> dead(work.ops.size(), 0);
        for (size_t k = 0; k < work.ops.size(); ++k) {
            const GOp q = work.ops[k];
            if (q.type != OpType::QELEM || q.inputs.size() != 2 ||
                (q.mode != "QADD" && q.mode != "QFUSE_ADD_RELU"))
                continue;
            for (int side = 0; side < 2; ++side) {
                const int t = q.inputs[side];
                const int j = producer[t];
                if (j < 0 || dead[j] || work.ops[j].type != OpType::CONV ||
                    work.ops[j].mode != "IDENTITY" || !work.ops[j].fuse_mode.empty() ||
                    uses[t] != 1 || work.tensors[t].is_output)
                    continue;
                GOp f = work.ops[j];
                f.name = work.ops[j].name + "+" + q.name;
                f.fuse_mode = q.mode;
                f.mid_scale = work.tensors[t].scale;
                f.inputs = {work.ops[j].inputs[0], q.inputs[1 - side]};
                f.output = q.output;
                GWeight wm;
                wm.name = f.name + ":mid_scale";
                wm.dtype = fb::Float32;
                wm.scale = f.mid_scale;  // read by the kernel stub from the tensor struct
                wm.dims = {1};
                wm.data.assign((const uint8_t*)&f.mid_scale, (const uint8_t*)&f.mid_scale + 4);
                wm.use_count = 1;
                work.weights.push_back(std::move(wm));
                f.mid_weight = (int)work.weights.size() - 1;
                work.ops[k] = f;
                dead[j] = 1;
                break;
            }
        }
        std::vector<GOp> kept;
        for (size_t k = 0; k < work.ops.size(); ++k)
            if (!dead[k])
                kept.push_back(work.ops[k]);
        work.ops = kept;
    }

    // ---- fusion: a first-layer ConvBias whose only consumer is a MAX pooling 3x3 / 2 / pad 1
    // becomes one instruction (the ResNet stem), where the kernel pack takes the fused
    // operator at every batch size of the model ----
    if (g->fuse_conv_pooling) {
        std::vector<int> uses(work.tensors.size(), 0), producer(work.tensors.size(), -1);
        for (size_t k = 0; k < work.ops.size(); ++k) {
            for (int id : work.ops[k].inputs)
                uses[id]++;
            producer[work.ops[k].output] = (int)k;
        }
        std::vector<char> dead(work.ops.size(), 0);
        for (size_t k = 0; k < work.ops.size(); ++k) {
            const GOp q = work.ops[k];
            if (q.type != OpType::POOL || q.f32 || q.mode != "MAX" || q.kh != 3 || q.kw != 3 ||
                q.stride != 2 || q.pad != 1)
                continue;
            const int t = q.inputs[0];
            const int j = producer[t];
            if (j < 0 || dead[j] || work.ops[j].type != OpType::CONV || work.ops[j].f32 ||
                !work.ops[j].fuse_mode.empty() || uses[t] != 1 || work.tensors[t].is_output)
                continue;
            GOp f = work.ops[j];
            f.name = work.ops[j].name + "+" + q.name;
            f.pool_fused = true;
            f.output = q.output;
            bool ok = true;
            for (int b = 0; b < nr_batches && ok; ++b) {
                auto ctx = work.context_for(f, batches[b]);
                bool any = false;
                for (auto* kf : KernelGen::Cuda::ArchKernelPack::GetKernel(KernType::ConvKernel))
                    any = any || kf->IsAvailable(ctx.get());
                ok = any;
            }
            if (!ok)
                continue;
            work.ops[k] = f;
            dead[j] = 1;
        }
        std::vector<GOp> kept;
        for (size_t k = 0; k < work.ops.size(); ++k)
            if (!dead[k])
                kept.push_back(work.ops[k]);
        work.ops = kept;
    }

    // ---- tensors that no instruction touches any more (the inner results of fused pairs)
    // leave the model: they would be listed with their full size and no place in the arena ----
    {
        std::vector<char> used(work.tensors.size(), 0);
        for (size_t i = 0; i < work.tensors.size(); ++i)
            used[i] = work.tensors[i].is_input || work.tensors[i].is_output;
        for (auto& op : work.ops) {
            for (int id : op.inputs)
                used[id] = 1;
            used[op.output] = 1;
        }
        std::vector<int> remap(work.tensors.size(), -1);
        std::vector<GTensor> kept;
        for (size_t i = 0; i < work.tensors.size(); ++i)
            if (used[i]) {
                remap[i] = (int)kept.size();
                kept.push_back(work.tensors[i]);
            }
        for (auto& op : work.ops) {
            for (int& id : op.inputs)
                id = remap[id];
            op.output = remap[op.output];
        }
        work.tensors = kept;
    }

    // ---- kernel selection (first available kernel of the CUDA pack wins) ----
    std::vector<std::string> op_symbol(work.ops.size());
    std::map<std::string, int> kernel_id;
    for (size_t k = 0; k < work.ops.size(); ++k) {
        const GOp& op = work.ops[k];
        auto ctx = work.context_for(op, batches[0]);
        const KernelGen::KernelFunc* chosen = nullptr;
        for (auto* kf : KernelGen::Cuda::ArchKernelPack::GetKernel(mb200c_graph::kern_type(op.type)))
            if (kf->IsAvailable(ctx.get())) {
                chosen = kf;
                break;
            }
        if (!chosen)
            return err("no CUDA kernel is available for operator '%s'", op.name.c_str());
        const std::string sym = chosen->GetKernelSymbol(ctx.get());
        op_symbol[k] = sym;
        if (!kernel_id.count(sym)) {
            kernel_id[sym] = (int)g->symbols.size();
            g->symbols.push_back(sym);
            g->kernel_of[sym] = chosen;
            g->ctx_of[sym] = ctx;
        }
    }

    // ---- weights ----
    std::vector<fb::NodeP> wnodes;
    for (auto& w : work.weights) {
        auto n = fb::make_table();
        n->add_ref(fb::field::W_dtype, dtype_node(w.dtype, w.scale));
        n->add_ref(fb::field::W_layout, layout_node(w.dims, contiguous(w.dims), fb::NCHW));
        n->add<int32_t>(fb::field::W_use_count, w.use_count);
        n->add_ref(fb::field::W_data, fb::make_bytes(w.data.data(), w.data.size()));
        n->add_ref(fb::field::W_name, fb::make_string(w.name));
        wnodes.push_back(n);
    }

    // ---- one DeviceModel per batch size ----
    std::vector<fb::NodeP> dmodels;
    for (int bi = 0; bi < nr_batches && g->bare_metal_model != 2; ++bi) {
        const int batch = batches[bi];
        if (batch <= 0)
            return err("compile: batch %d", batch);
        // workspace bytes per operator, as the kernel that was selected reports them
        std::vector<size_t> ws_bytes(work.ops.size(), 0), ws_offsets;
        for (size_t k = 0; k < work.ops.size(); ++k) {
            auto* with_ws =
                    dynamic_cast<const KernelGen::Cuda::WithWorkspace*>(g->kernel_of[op_symbol[k]]);
            if (!with_ws)
                continue;
            auto ctx = work.context_for(work.ops[k], batch);
            ws_bytes[k] = with_ws->WorkspaceBytes(ctx.get());
        }
        std::vector<size_t> offsets;
        Compiled c;
        c.arena = plan_memory(work, work.ops, batch, ws_bytes, &offsets, &ws_offsets, &c.unplanned);
        g->compiled.push_back(c);

        std::vector<fb::NodeP> tnodes;
        std::vector<int> use_count(work.tensors.size(), 0);
        for (auto& op : work.ops)
            for (int id : op.inputs)
                use_count[id]++;
        for (size_t i = 0; i < work.tensors.size(); ++i) {
            const GTensor& t = work.tensors[i];
            const std::vector<int> dims = t.nchw44 ? std::vector<int>{batch, t.c / 4, t.h, t.w, 4}
                                                   : std::vector<int>{batch, t.c, t.h, t.w};
            const std::vector<int> stride =
                    t.nchw || t.nchw44 ? contiguous(dims)
                                       : std::vector<int>{t.h * t.w * t.c, 1, t.w * t.c, t.c};
            auto n = fb::make_table();
            n->add_ref(fb::field::T_dtype, dtype_node(t.f32 ? fb::Float32 : fb::QInt8, t.scale));
            n->add_ref(fb::field::T_layout,
                       layout_node(dims, stride,
                                   t.nchw44 ? fb::NCHW4 : t.nchw ? fb::NCHW : fb::NHWC));
            n->add<int64_t>(fb::field::T_offset, (int64_t)offsets[i]);
            n->add<int32_t>(fb::field::T_use_count, use_count[i]);
            n->add_ref(fb::field::T_name, fb::make_string(t.name));
            tnodes.push_back(n);
        }
        std::vector<fb::NodeP> inodes;
        std::vector<uint8_t> itags;
        for (size_t k = 0; k < work.ops.size(); ++k) {
            const GOp& op = work.ops[k];
            std::vector<int32_t> in;
            std::vector<int8_t> in_t;
            if (op.type == OpType::MATMUL) {
                in.push_back(op.inputs[0]);
                in_t.push_back(fb::TENSOR);
                in.push_back(op.weights[0]);
                in_t.push_back(fb::WEIGHT);
            } else if (op.type == OpType::CONV) {
                // operand order src, filter, [bias], [channel scales], [z, mid scale]
                in.push_back(op.inputs[0]);
                in_t.push_back(fb::TENSOR);
                for (int wid : op.weights) {
                    in.push_back(wid);
                    in_t.push_back(fb::WEIGHT);
                }
                if (!op.fuse_mode.empty()) {
                    in.push_back(op.inputs[1]);
                    in_t.push_back(fb::TENSOR);
                    in.push_back(op.mid_weight);
                    in_t.push_back(fb::WEIGHT);
                } else if (op.f32 && op.inputs.size() > 1) {
                    in.push_back(op.inputs[1]);  // z: added after the activation
                    in_t.push_back(fb::TENSOR);
                }
            } else {
                for (int id : op.inputs) {
                    in.push_back(id);
                    in_t.push_back(fb::TENSOR);
                }
            }
            auto ws = fb::make_table();
            ws->add<int64_t>(fb::field::WS_size, (int64_t)ws_bytes[k]);
            ws->add<int64_t>(fb::field::WS_offset, (int64_t)ws_offsets[k]);
            auto n = fb::make_table();
            n->add_ref(fb::field::O_name, fb::make_string(op.name));
            n->add_ref(fb::field::O_type, fb::make_string(op_symbol[k]));
            n->add_ref(fb::field::O_inputs, fb::make_vec<int32_t>(in));
            n->add_ref(fb::field::O_input_types, fb::make_vec<int8_t>(in_t));
            n->add_ref(fb::field::O_outputs, fb::make_vec<int32_t>({op.output}));
            n->add_ref(fb::field::O_workspace, ws);
            n->add<int32_t>(fb::field::O_init_id, kernel_id[op_symbol[k]]);
            n->add<int32_t>(fb::field::O_kernel_id, kernel_id[op_symbol[k]]);
            n->add<int32_t>(fb::field::O_workspace_id, kernel_id[op_symbol[k]]);
            n->add<int32_t>(fb::field::O_deduce_id, -1);
            inodes.push_back(n);
            itags.push_back(fb::INST_OPR);
        }
        std::vector<int32_t> ins, outs;
        for (size_t i = 0; i < work.tensors.size(); ++i) {
            if (work.tensors[i].is_input)
                ins.push_back((int)i);
            if (work.tensors[i].is_output)
                outs.push_back((int)i);
        }
        if (outs.empty())
            return err("compile: the graph has no output");
        auto dm = fb::make_table();
        dm->add<int8_t>(fb::field::D_device, (int8_t)fb::CUDA_SM100);
        dm->add_ref(fb::field::D_tensor_pool, fb::make_table_vec(tnodes));
        dm->add_ref(fb::field::D_instructions_type, fb::make_vec<uint8_t>(itags));
        dm->add_ref(fb::field::D_instructions, fb::make_table_vec(inodes));
        dm->add<uint64_t>(fb::field::D_tensor_memory, (uint64_t)c.arena);
        dm->add_ref(fb::field::D_inputs, fb::make_vec<int32_t>(ins));
        dm->add_ref(fb::field::D_outputs, fb::make_vec<int32_t>(outs));
        dmodels.push_back(dm);
    }
    // ---- the same network for the reference's C runtime: a BARE_METAL DeviceModel per batch
    // whose Oprs name the reference's own kernels (one operator each, NCHW tensors, the
    // weights of the shared pool as they are). runtime/schema/model.fbs:391 allows several
    // DeviceModels; runtime/src/parse.c:470-520 takes those of the devices it knows. ----
    for (int bi = 0; bi < nr_batches && g->bare_metal_model != 0; ++bi) {
        const int batch = batches[bi];
        if (batch <= 0)
            return err("compile: batch %d", batch);
        mb200c_graph bm = *g;  // the operators as the user added them: no relayout, no fusion
        for (auto& t : bm.tensors)
            t.nchw = true;
        std::vector<std::string> sym(bm.ops.size());
        std::map<std::string, int> bm_id;
        for (size_t k = 0; k < bm.ops.size(); ++k) {
            const GOp& op = bm.ops[k];
            const bool known = !op.f32 && !op.flt44 &&
                               ((op.type == OpType::CONV && op.weights.size() <= 2 &&
                                 (op.weights.size() == 1 || op.has_bias)) ||
                                op.type == OpType::POOL || op.type == OpType::QELEM);
            if (!known)
                return err("operator '%s' has no BARE_METAL form here (qint8 ConvBias with "
                           "per-tensor scales, Pooling and ElemwiseMultiType do)", op.name.c_str());
            auto ctx = bm.context_for(op, batch);
            const KernelGen::KernelFunc* kf = nullptr;
            for (auto* c : KernelGen::Cuda::ArchKernelPack::GetKernel(mb200c_graph::kern_type(op.type)))
                if (c->IsAvailable(ctx.get())) {
                    kf = c;
                    break;
                }
            if (!kf)
                return err("operator '%s' is not admitted", op.name.c_str());
            // the reference's symbol for the same operator: its own prefix and format name
            std::string s = kf->GetKernelSymbol(ctx.get());
            const std::string prefix = "cuda_sm100_";
            if (s.compare(0, prefix.size(), prefix) != 0)
                return err("unexpected symbol %s", s.c_str());
            s = "kernel_" + s.substr(prefix.size());
            const size_t at = s.find("_NHWC_");
            if (at != std::string::npos)
                s.replace(at, 6, "_NCHW_");
            sym[k] = s;
            if (!bm_id.count(s)) {
                const int id = (int)bm_id.size();
                bm_id[s] = id;
            }
        }
        std::vector<size_t> no_ws(bm.ops.size(), 0), offsets, ws_offsets;
        size_t unplanned = 0;
        const size_t arena = plan_memory(bm, bm.ops, batch, no_ws, &offsets, &ws_offsets, &unplanned);
        std::vector<int> use_count(bm.tensors.size(), 0);
        for (auto& op : bm.ops)
            for (int id : op.inputs)
                use_count[id]++;
        std::vector<fb::NodeP> tnodes, inodes;
        std::vector<uint8_t> itags;
        for (size_t i = 0; i < bm.tensors.size(); ++i) {
            const GTensor& t = bm.tensors[i];
            const std::vector<int> dims = {batch, t.c, t.h, t.w};
            auto n = fb::make_table();
            n->add_ref(fb::field::T_dtype, dtype_node(fb::QInt8, t.scale));
            n->add_ref(fb::field::T_layout, layout_node(dims, contiguous(dims), fb::NCHW));
            n->add<int64_t>(fb::field::T_offset, (int64_t)offsets[i]);
            n->add<int32_t>(fb::field::T_use_count, use_count[i]);
            n->add_ref(fb::field::T_name, fb::make_string(t.name));
            tnodes.push_back(n);
        }
        for (size_t k = 0; k < bm.ops.size(); ++k) {
            const GOp& op = bm.ops[k];
            std::vector<int32_t> in;
            std::vector<int8_t> in_t;
            for (int id : op.inputs) {
                in.push_back(id);
                in_t.push_back(fb::TENSOR);
            }
            if (op.type == OpType::CONV) {
                // src, filter, [bias]
                in.resize(1);
                in_t.resize(1);
                for (int wid : op.weights) {
                    in.push_back(wid);
                    in_t.push_back(fb::WEIGHT);
                }
            }
            auto ws = fb::make_table();
            ws->add<int64_t>(fb::field::WS_size, 0);
            ws->add<int64_t>(fb::field::WS_offset, 0);
            auto n = fb::make_table();
            n->add_ref(fb::field::O_name, fb::make_string(op.name));
            n->add_ref(fb::field::O_type, fb::make_string(sym[k]));
            n->add_ref(fb::field::O_inputs, fb::make_vec<int32_t>(in));
            n->add_ref(fb::field::O_input_types, fb::make_vec<int8_t>(in_t));
            n->add_ref(fb::field::O_outputs, fb::make_vec<int32_t>({op.output}));
            n->add_ref(fb::field::O_workspace, ws);
            n->add<int32_t>(fb::field::O_init_id, bm_id[sym[k]]);
            n->add<int32_t>(fb::field::O_kernel_id, bm_id[sym[k]]);
            n->add<int32_t>(fb::field::O_workspace_id, bm_id[sym[k]]);
            n->add<int32_t>(fb::field::O_deduce_id, -1);
            inodes.push_back(n);
            itags.push_back(fb::INST_OPR);
        }
        std::vector<int32_t> ins, outs;
        for (size_t i = 0; i < bm.tensors.size(); ++i) {
            if (bm.tensors[i].is_input)
                ins.push_back((int)i);
            if (bm.tensors[i].is_output)
                outs.push_back((int)i);
        }
        if (outs.empty())
            return err("compile: the graph has no output");
        auto dm = fb::make_table();
        dm->add<int8_t>(fb::field::D_device, (int8_t)fb::BARE_METAL);
        dm->add_ref(fb::field::D_tensor_pool, fb::make_table_vec(tnodes));
        dm->add_ref(fb::field::D_instructions_type, fb::make_vec<uint8_t>(itags));
        dm->add_ref(fb::field::D_instructions, fb::make_table_vec(inodes));
        dm->add<uint64_t>(fb::field::D_tensor_memory, (uint64_t)arena);
        dm->add_ref(fb::field::D_inputs, fb::make_vec<int32_t>(ins));
        dm->add_ref(fb::field::D_outputs, fb::make_vec<int32_t>(outs));
        dmodels.push_back(dm);
    }
    auto model = fb::make_table();
    model->add_ref(fb::field::M_weight_pool, fb::make_table_vec(wnodes));
    model->add_ref(fb::field::M_device_models, fb::make_table_vec(dmodels));
    model->add<uint8_t>(fb::field::M_const_shape, 1);
    model->add_ref(fb::field::M_name, fb::make_string(g->name));
    fb::Writer w;
    g->bytes = w.finish(model);
    g->symbols_joined.clear();
    for (auto& s : g->symbols)
        g->symbols_joined += s + "\n";
    *bytes = g->bytes.data();
    *len = g->bytes.size();
    return 0;
}

const char* mb200c_kernel_symbols(mb200c_graph* g) {
    return g ? g->symbols_joined.c_str() : "";
}

size_t mb200c_arena_bytes(mb200c_graph* g, int i) {
    return g && i >= 0 && (size_t)i < g->compiled.size() ? g->compiled[i].arena : 0;
}

size_t mb200c_unplanned_bytes(mb200c_graph* g, int i) {
    return g && i >= 0 && (size_t)i < g->compiled.size() ? g->compiled[i].unplanned : 0;
}

int mb200c_export_kernels(mb200c_graph* g, const char* dir) {
    if (!g || !dir)
        return err("export_kernels: bad argument");
    if (g->symbols.empty())
        return err("export_kernels: compile the graph first");
    const std::string d = dir;
    // kernels.h / kernels.c follow the shape of the reference exporter's output
    // (compiler/lib/Target/TinyNN/KernelExporter.cpp:15-66): function tables indexed by
    // kernel_id / init_id and a loader that fills them.
    std::ofstream h(d + "/kernels.h"), c(d + "/kernels.c");
    if (!h || !c)
        return err("export_kernels: cannot write into %s", dir);
    const size_t n = g->symbols.size();
    h << "#ifndef KERNELS_H\n#define KERNELS_H\n#include \"megcc_b200_runtime.h\"\n"
      << "#define NR_KERNELS (" << n << ")\n#define NR_INIT (" << n << ")\n"
      << "extern KernelFunc kernels[NR_KERNELS];\nextern InitFunc init_kernels[NR_INIT];\n"
      << "extern WorkspaceFunc workspace_func[NR_KERNELS];\n"
      << "void load_kernel_init_function(void);\n";
    c << "#include \"kernels.h\"\nKernelFunc kernels[NR_KERNELS];\nInitFunc init_kernels[NR_INIT];\n"
      << "WorkspaceFunc workspace_func[NR_KERNELS];\n";
    std::stringstream loader;
    loader << "void load_kernel_init_function(void) {\n";
    for (size_t i = 0; i < n; ++i) {
        const std::string& sym = g->symbols[i];
        const KernelGen::KernelFunc* kf = g->kernel_of[sym];
        TContext* ctx = g->ctx_of[sym].get();
        h << "TinyNNStatus " << kf->GetKernelSignature(ctx) << ";\n"
          << "TinyNNStatus " << kf->GetInitSignature(ctx) << ";\n"
          << "TinyNNStatus " << kf->GetWorkspaceSignature(ctx) << ";\n";
        loader << "    kernels[" << i << "] = " << sym << ";\n    init_kernels[" << i
               << "] = " << kf->GetInitSymbol(ctx) << ";\n    workspace_func[" << i
               << "] = " << kf->GetWorkspaceSymbol(ctx) << ";\n";
        std::ofstream k(d + "/" + sym + ".c");
        if (!k)
            return err("export_kernels: cannot write %s.c", sym.c_str());
        const std::string body = kf->GetKernelBody(ctx);
        std::string init = kf->GetInitBody(ctx);
        k << kf->GetBodyGuardBegin(ctx) << "#include \"kernels.h\"\n" << body << "\n" << init
          << "\n" << kf->GetWorkspaceBody(ctx) << "\n" << kf->GetBodyGuardEnd(ctx);
    }
    loader << "}\n";
    c << loader.str();
    h << "#endif\n";
    return 0;
}

int mb200c_probe_conv_symbol(
        int ic, int oc, int h, int w, int k, int stride, int pad, int groups, const char* nonline,
        int with_bias, const char* format, char* symbol_out, size_t symbol_cap) {
    CodeGenContext ctx;
    set_u32(ctx, "kernel_h", k);
    set_u32(ctx, "kernel_w", k);
    set_u32(ctx, "stride_h", stride);
    set_u32(ctx, "stride_w", stride);
    set_u32(ctx, "pad_h", pad);
    set_u32(ctx, "pad_w", pad);
    set_u32(ctx, "dilate_h", 1);
    set_u32(ctx, "dilate_w", 1);
    set_str(ctx, "sparse", groups == 1 ? "DENSE" : "GROUP");
    set_str(ctx, "format", format ? format : "NCHW");
    set_str(ctx, "mode", "CROSS_CORRELATION");
    set_str(ctx, "nonlineMode", nonline ? nonline : "IDENTITY");
    set_opr(ctx, "operand:0", operand("qsi8", {1, (size_t)ic, (size_t)h, (size_t)w}, 1.f));
    if (groups == 1)
        set_opr(ctx, "operand:1", operand("qsi8", {(size_t)oc, (size_t)ic, (size_t)k, (size_t)k}, 1.f));
    else
        set_opr(ctx, "operand:1",
                operand("qsi8", {(size_t)groups, (size_t)oc / groups, (size_t)ic / groups,
                                 (size_t)k, (size_t)k}, 1.f));
    set_opr(ctx, "operand:2",
            with_bias ? operand("qsi32", {1, (size_t)oc, 1, 1}, 1.f) : operand("qsi32", {}, 1.f));
    set_opr(ctx, "operand:3", operand("qsi8", {1, (size_t)oc, (size_t)h, (size_t)w}, 1.f));
    set_i32(ctx, "nr_operands", 4);
    for (auto* kf : KernelGen::Cuda::ArchKernelPack::GetKernel(KernType::ConvKernel))
        if (kf->IsAvailable(&ctx)) {
            const std::string s = kf->GetKernelSymbol(&ctx);
            if (symbol_out && symbol_cap)
                snprintf(symbol_out, symbol_cap, "%s", s.c_str());
            return 1;
        }
    return 0;
}

}  // extern "C"
