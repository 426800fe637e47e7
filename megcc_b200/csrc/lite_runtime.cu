// The runtime behind the LITE_* C API: loads a tinynn model whose DeviceModel targets
// CUDA_SM100, lays every tensor into one device arena at the offsets the compile-time
// planner chose, and replays the instruction list as one CUDA graph on one stream.
//
// It takes the place of the reference's parse.c / init.c / vm.c / vm/op.c / lite/*.c
// (runtime/src): same model format, same structs handed to kernels, same status codes.
//
// Dispatch follows the reference (runtime/src/vm/op.c:161-163): every Opr is executed as
// kernels[opr->kernel_id](inputs, nr_input, outputs, nr_output, &workspace, &opt) through a
// table of the reference's uniform KernelFunc type, and its weights are preprocessed through
// init_kernels[opr->init_id] with the three-phase protocol of runtime/src/init.c:29-131.
// The tables come from the generated kernels.c of the compile side when the caller registered
// one (mb200_lite_set_kernel_tables); entries nobody registered are filled once at load time
// with the library's own implementations, selected by the Opr's symbol.
#include <algorithm>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/megcc_b200.h"
#include "../../include/megcc_b200_lite.h"
#include "../../include/megcc_b200_runtime.h"
#include "internal.h"
#include "tinynn_format.h"

namespace fb = tinynn_fb;
using mb200::set_error;

namespace {

LiteLogLevel g_log_level = LITE_WARN;

void log_at(LiteLogLevel lvl, const char* fmt, ...) {
    if (lvl < g_log_level)
        return;
    static const char* tag[] = {"DEBUG", "INFO", "WARN", "ERROR"};
    fprintf(stderr, "megcc_b200 %s: ", tag[lvl]);
    va_list ap;
    va_start(ap, fmt);
    vfprintf(stderr, fmt, ap);
    va_end(ap);
}

size_t dtype_bytes(TinyNNDType t) {
    switch (t) {
        case TinyNN_FLOAT:
        case TinyNN_INT:
        case TinyNN_QINT32:
            return 4;
        case TinyNN_FLOAT16:
        case TinyNN_INT16:
            return 2;
        default:
            return 1;
    }
}

// bytes of a tensor, or SIZE_MAX when the product of its extents does not fit a size_t
size_t tensor_bytes(const Tensor& t) {
    size_t n = dtype_bytes(t.dtype.type_enum);
    for (int i = 0; i < t.layout.nr_dim; ++i) {
        const size_t d = t.layout.dims[i];
        if (d != 0 && n > (SIZE_MAX / 4) / d)
            return SIZE_MAX;
        n *= d;
    }
    return n;
}

enum OpKind {
    OP_CONV, OP_POOL, OP_QELEM, OP_TYPECVT, OP_RELAYOUT_TO_NHWC, OP_RELAYOUT_TO_NCHW, OP_MATMUL,
    // fp32 path
    OP_CONV_F32, OP_MATMUL_F32, OP_ELEM_F32, OP_CONCAT_F32, OP_FOCUS_F32, OP_RESIZE_F32,
    OP_POOL_F32, OP_RELAYOUT_F32_TO_NHWC, OP_RELAYOUT_F32_TO_NCHW, OP_RELAYOUT_44_TO_NHWC,
    OP_RELAYOUT_NHWC_TO_44,
    // a symbol this library has no implementation for: runs only through a registered table
    OP_EXTERNAL
};

struct OpPlan {
    OpKind kind;
    std::string symbol, name;
    // attributes baked into the symbol
    int kh = 0, kw = 0, sh = 1, sw = 1, ph = 0, pw = 0, dh = 1, dw = 1;
    bool dense = true, has_bias = false;
    int mode = 0;  // nonline / pooling mode / elemwise mode
    std::vector<Tensor*> inputs, outputs;
    std::vector<int> weight_inputs;  // indices (into inputs) that are weights
    Workspace ws{nullptr, 0, 0};
    bool needs_init = false;
    int pool = 0;          // ConvBias with the MAX pooling 3x3 / 2 / pad 1 behind it folded in
    int flt44 = 0;         // filter layout: 0 OIHW, 1 / 2 / 3 NCHW44 dense / channel-wise / first layer
    int z_mode = 0;        // fused elemwise step: 0 none, else MB200_QADD + 1 / MB200_QFUSE_ADD_RELU + 1
    bool f32_z = false;    // fp32 ConvBias with a tensor added after the activation
    int oc = 0, icpg = 0;  // fp32 ConvBias: output channels, input channels per group (symbol)
    // table indices from the model file and the functions they resolved to
    int kernel_id = -1, init_id = -1;
    KernelFunc kernel_fn = nullptr;
    InitFunc init_fn = nullptr;
    float ms_total = 0;
    int ms_count = 0;
};

struct MemForwardPlan {
    Tensor* in;
    Tensor* out;
    int offset;
};

struct Instr {
    bool is_opr;
    OpPlan op;
    MemForwardPlan mf;
};

constexpr size_t kArenaSlack = 131072 + 4096;

struct Arena {
    void* ptr = nullptr;
    size_t bytes = 0;
    int device = 0;
    ~Arena() {
        if (ptr) {
            mb200_unregister_readable_range(ptr);
            cudaSetDevice(device);
            cudaFree(ptr);
        }
    }
};

struct IoSlot {
    Tensor* tensor = nullptr;
    void* user_ptr = nullptr;   // what LITE_reset_tensor_memory was given (inputs)
    bool user_is_device = false;
    bool want_device = false;   // LiteIO.is_host == 0
    void* host_stage = nullptr; // pinned copy of an output
    size_t bytes = 0;
};

struct DevModel {
    std::vector<Tensor> tensors;
    std::vector<std::string> names;
    std::vector<Instr> instrs;
    std::vector<IoSlot> inputs, outputs;
    size_t tensor_memory = 0;
    // instantiated graphs, one per set of input addresses (device pointers are baked into the
    // captured kernels): a caller that cycles a few device buffers replays, it does not
    // re-capture. Most recently used first, at most kMaxGraphs.
    struct CapturedGraph {
        std::vector<void*> inputs;
        cudaGraphExec_t exec;
    };
    static constexpr size_t kMaxGraphs = 4;
    std::vector<CapturedGraph> graphs;
    bool memory_ready = false;
    bool ran_eager = false;
};

struct Network;

struct IoHandle {
    Network* net;
    bool is_input;
    int index;
};

struct Network {
    LiteConfig config;
    std::vector<std::string> io_device_names;  // outputs/inputs declared is_host == 0
    int device_id = 0;
    cudaStream_t stream = nullptr;
    Device device{256, TinyNN_CUDA_SM100, nullptr, nullptr};
    RuntimeOpt opt{nullptr, nullptr, 0, nullptr};
    std::vector<uint8_t> owned_model;  // LITE_load_model_from_path
    std::vector<Tensor> weights;       // device-resident
    std::vector<std::string> weight_names;
    std::vector<const uint8_t*> weight_host;  // into the model buffer, until uploaded
    std::vector<Tensor> processed;     // packed filters
    // function tables of a generated kernels.c, when the caller registered one
    std::vector<KernelFunc> ext_kernels;
    std::vector<InitFunc> ext_inits;
    void* weight_arena = nullptr;
    std::vector<DevModel> models;
    int active = 0;
    std::shared_ptr<Arena> arena = std::make_shared<Arena>();
    size_t arena_need = 0;
    bool loaded = false, pending = false, use_graph = true, profile = false;
    std::vector<std::unique_ptr<IoHandle>> handles;
    // Large host inputs are copied in as several pieces on side streams: one copy stream
    // measured 40 GB/s over PCIe gen5 x16, four concurrent pieces 54 GB/s.
    static constexpr int kCopyStreams = 3;
    cudaStream_t copy_stream[kCopyStreams] = {nullptr, nullptr, nullptr};
    cudaEvent_t copy_fork = nullptr, copy_join[kCopyStreams] = {nullptr, nullptr, nullptr};
};

// Networks on one device run their instruction sequences one after the other, in the order of
// the LITE_forward calls, while their input and output copies overlap the other networks'
// kernels: every kernel here is a persistent grid sized for the whole GPU, and two such
// sequences side by side only take turns at kernel granularity with late-starting CTAs
// (measured slower than back to back). One event per device carries the order; the mutex
// keeps wait - launch - record of one network together when several host threads call
// LITE_forward. MB200_LITE_SERIAL_COMPUTE=0 switches the ordering off.
struct ComputeLane {
    std::mutex mu;
    cudaEvent_t done = nullptr;
    bool recorded = false;
};
// Defaults of a new network, taken from the environment once per process
// (MB200_NO_GRAPH=1, MB200_PROFILE=1, MB200_LITE_SERIAL_COMPUTE=0); a network's own settings
// change through mb200_lite_set_option afterwards.
struct RuntimeDefaults {
    bool use_graph = true, profile = false, serial_compute = true;
};
const RuntimeDefaults& runtime_defaults() {
    static const RuntimeDefaults d = [] {
        RuntimeDefaults v;
        const char* e = getenv("MB200_NO_GRAPH");
        v.use_graph = !(e && e[0] == '1');
        e = getenv("MB200_PROFILE");
        v.profile = e && e[0] == '1';
        e = getenv("MB200_LITE_SERIAL_COMPUTE");
        v.serial_compute = !(e && atoi(e) == 0);
        return v;
    }();
    return d;
}

ComputeLane* compute_lane(int device) {
    static ComputeLane lanes[64];
    const bool enabled = runtime_defaults().serial_compute;
    if (!enabled || device < 0 || device >= 64)
        return nullptr;
    return &lanes[device];
}

// Host -> device copy of one input, ordered after what `net->stream` holds so far and before
// what it is given next. Pieces of at least 2 MiB go to the side streams.
cudaError_t copy_input(Network* net, void* dst, const void* src, size_t bytes) {
    constexpr size_t kMinPiece = 2u << 20;
    const int pieces = bytes >= 4 * kMinPiece ? Network::kCopyStreams + 1 : 1;
    if (pieces == 1)
        return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, net->stream);
    cudaError_t e;
    if (!net->copy_fork) {
        if ((e = cudaEventCreateWithFlags(&net->copy_fork, cudaEventDisableTiming)) != cudaSuccess)
            return e;
        for (int i = 0; i < Network::kCopyStreams; ++i) {
            if ((e = cudaStreamCreateWithFlags(&net->copy_stream[i], cudaStreamNonBlocking)) !=
                        cudaSuccess ||
                (e = cudaEventCreateWithFlags(&net->copy_join[i], cudaEventDisableTiming)) !=
                        cudaSuccess)
                return e;
        }
    }
    const size_t piece = (bytes / pieces + 255) / 256 * 256;
    if ((e = cudaEventRecord(net->copy_fork, net->stream)) != cudaSuccess)
        return e;
    size_t off = 0;
    for (int i = 0; i < Network::kCopyStreams && off < bytes; ++i) {
        const size_t len = bytes - off < piece ? bytes - off : piece;
        if ((e = cudaStreamWaitEvent(net->copy_stream[i], net->copy_fork, 0)) != cudaSuccess ||
            (e = cudaMemcpyAsync((uint8_t*)dst + off, (const uint8_t*)src + off, len,
                                 cudaMemcpyHostToDevice, net->copy_stream[i])) != cudaSuccess ||
            (e = cudaEventRecord(net->copy_join[i], net->copy_stream[i])) != cudaSuccess)
            return e;
        off += len;
    }
    if (off < bytes &&
        (e = cudaMemcpyAsync((uint8_t*)dst + off, (const uint8_t*)src + off, bytes - off,
                             cudaMemcpyHostToDevice, net->stream)) != cudaSuccess)
        return e;
    for (int i = 0; i < Network::kCopyStreams; ++i)
        if ((e = cudaStreamWaitEvent(net->stream, net->copy_join[i], 0)) != cudaSuccess)
            return e;
    return cudaSuccess;
}

thread_local char g_lite_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_lite_err, sizeof(g_lite_err), fmt, ap);
    va_end(ap);
    log_at(LITE_ERROR, "%s\n", g_lite_err);
    return code;
}

int cuda_fail(cudaError_t e, const char* what) {
    return fail(TinyNN_ERROR_RUNTIME, "%s: %s", what, cudaGetErrorString(e));
}

// ---------------------------------------------------------------------------------------
// symbol -> plan
// ---------------------------------------------------------------------------------------
bool ends_with(const std::string& s, const char* suf) {
    const size_t n = strlen(suf);
    return s.size() >= n && s.compare(s.size() - n, n, suf) == 0;
}

bool parse_symbol(const std::string& sym, OpPlan* op) {
    op->symbol = sym;
    if (sym.compare(0, 18, "cuda_sm100_conv2d_") == 0) {
        char sparse[16] = {0}, format[16] = {0};
        int used = 0;
        if (sscanf(sym.c_str(),
                   "cuda_sm100_conv2d_%dx%d_%15[A-Z0-9]_%15[A-Z]_p%dx%d_s%dx%d_d%dx%d_%n", &op->kh,
                   &op->kw, format, sparse, &op->ph, &op->pw, &op->sh, &op->sw, &op->dh, &op->dw,
                   &used) != 10 ||
            used == 0)
            return false;
        // activations are NHWC; NHWC44D / NHWC44C / NHWC44H say the filter arrives in the
        // dense / channel-wise / first-layer NCHW44 layout
        static const char* kFormats[] = {"NHWC", "NHWC44D", "NHWC44C", "NHWC44H"};
        op->flt44 = -1;
        for (int f = 0; f < 4; ++f)
            if (strcmp(format, kFormats[f]) == 0)
                op->flt44 = f;
        if (op->flt44 < 0)
            return false;
        op->dense = strcmp(sparse, "DENSE") == 0;
        if (!op->dense && strcmp(sparse, "GROUP") != 0)
            return false;
        std::string rest = sym.substr(used);
        int oc = 0, icpg = 0, used2 = 0;
        if ((sscanf(rest.c_str(), "oc%d_icpg%d_f32%n", &oc, &icpg, &used2) == 2 && used2 > 0) ||
            (icpg = 0, sscanf(rest.c_str(), "oc%d_f32%n", &oc, &used2) == 1 && used2 > 0)) {
            // fp32 ConvBias: ..._oc<N>[_icpg<M>]_f32[_bias][_ACT][_z_ADD]
            if (op->flt44)
                return false;
            op->kind = OP_CONV_F32;
            op->oc = oc;
            op->icpg = icpg;
            rest = rest.substr(used2);
            if (ends_with(rest, "_z_ADD")) {
                op->f32_z = true;
                rest.resize(rest.size() - strlen("_z_ADD"));
            }
            op->has_bias = rest.find("_bias") != std::string::npos;
            op->mode = ends_with(rest, "_H_SWISH")  ? MB200_F32_H_SWISH
                       : ends_with(rest, "_RELU")   ? MB200_F32_RELU
                       : ends_with(rest, "_SIGMOID") ? MB200_F32_SIGMOID
                       : ends_with(rest, "_SILU")   ? MB200_F32_SILU
                                                    : MB200_F32_IDENTITY;
            op->needs_init = true;
            return true;
        }
        op->kind = OP_CONV;
        if (rest.compare(0, 8, "qsi8qsi8") != 0)
            return false;
        // a MAX pooling 3x3 / 2 / pad 1 folded into the ConvBias is spelled last
        if (ends_with(rest, "_pool_MAX3x3s2p1")) {
            op->pool = 1;
            rest.resize(rest.size() - strlen("_pool_MAX3x3s2p1"));
        }
        // a fused elemwise step is spelled last: ..._z_QADD / ..._z_QFUSE_ADD_RELU
        if (ends_with(rest, "_z_QFUSE_ADD_RELU")) {
            op->z_mode = MB200_QFUSE_ADD_RELU + 1;
            rest.resize(rest.size() - strlen("_z_QFUSE_ADD_RELU"));
        } else if (ends_with(rest, "_z_QADD")) {
            op->z_mode = MB200_QADD + 1;
            rest.resize(rest.size() - strlen("_z_QADD"));
        }
        op->has_bias = rest.find("_bias") != std::string::npos;
        op->mode = ends_with(rest, "_H_SWISH") ? MB200_H_SWISH
                   : ends_with(rest, "_RELU")  ? MB200_RELU
                                               : MB200_IDENTITY;
        op->needs_init = true;
        return true;
    }
    if (sym.compare(0, 19, "cuda_sm100_pooling_") == 0) {
        const size_t p = sym.find("_NHWC_p");
        if (p == std::string::npos)
            return false;
        const std::string mode = sym.substr(19, p - 19);
        op->mode = mode == "MAX" ? 0 : mode == "AVERAGE" ? 1
                   : mode == "AVERAGE_COUNT_EXCLUDE_PADDING" ? 2 : -1;
        if (op->mode < 0)
            return false;
        if (sscanf(sym.c_str() + p, "_NHWC_p%dx%d_s%dx%d_w%dx%d_", &op->ph, &op->pw, &op->sh,
                   &op->sw, &op->kh, &op->kw) != 6)
            return false;
        op->kind = ends_with(sym, "_f32f32") ? OP_POOL_F32 : OP_POOL;
        return true;
    }
    if (sym.compare(0, 33, "cuda_sm100_elementwise_multitype_") == 0) {
        const size_t p = sym.find("_qsi8");
        if (p == std::string::npos)
            return false;
        const std::string mode = sym.substr(33, p - 33);
        op->mode = mode == "QADD" ? 0 : mode == "QFUSE_ADD_RELU" ? 1 : mode == "QMUL" ? 2
                   : mode == "QRELU" ? 3 : -1;
        op->kind = OP_QELEM;
        return op->mode >= 0;
    }
    if (sym.compare(0, 23, "cuda_sm100_elementwise_") == 0) {
        const size_t p = sym.find("_f32");
        if (p == std::string::npos)
            return false;
        const std::string mode = sym.substr(23, p - 23);
        static const struct { const char* name; int code; } kModes[] = {
                {"RELU", MB200_ELEM_RELU}, {"SIGMOID", MB200_ELEM_SIGMOID},
                {"SILU", MB200_ELEM_SILU}, {"H_SWISH", MB200_ELEM_H_SWISH},
                {"EXP", MB200_ELEM_EXP}, {"ADD", MB200_ELEM_ADD}, {"SUB", MB200_ELEM_SUB},
                {"MUL", MB200_ELEM_MUL}, {"MAX", MB200_ELEM_MAX},
                {"FUSE_ADD_RELU", MB200_ELEM_FUSE_ADD_RELU}};
        op->mode = -1;
        for (auto& m : kModes)
            if (mode == m.name)
                op->mode = m.code;
        op->kind = OP_ELEM_F32;
        return op->mode >= 0;
    }
    if (sym == "cuda_sm100_concat_NHWC_axis_1_f32") {
        op->kind = OP_CONCAT_F32;
        return true;
    }
    if (sym == "cuda_sm100_concat_focus_f32") {
        op->kind = OP_FOCUS_F32;
        return true;
    }
    if (sym == "cuda_sm100_resize_NHWC_NEAREST_f32") {
        op->kind = OP_RESIZE_F32;
        return true;
    }
    if (sym == "cuda_sm100_matmul_nn_qsi8qsi8qsi32_typecvt_qsi8") {
        op->kind = OP_MATMUL;
        op->needs_init = true;  // B [K][N] is re-laid to [N][K]
        return true;
    }
    if (sym == "cuda_sm100_matmul_nn_f32f32f32") {
        op->kind = OP_MATMUL_F32;
        op->needs_init = true;
        return true;
    }
    if (sym == "cuda_sm100_typecvt_qsi32qsi8") {
        op->kind = OP_TYPECVT;
        return true;
    }
    if (sym.compare(0, 30, "cuda_sm100_relayout_NCHW_NHWC_") == 0) {
        op->kind = ends_with(sym, "f32f32") ? OP_RELAYOUT_F32_TO_NHWC : OP_RELAYOUT_TO_NHWC;
        return true;
    }
    if (sym.compare(0, 32, "cuda_sm100_relayout_NCHW44_NHWC_") == 0) {
        op->kind = OP_RELAYOUT_44_TO_NHWC;
        return true;
    }
    if (sym.compare(0, 32, "cuda_sm100_relayout_NHWC_NCHW44_") == 0) {
        op->kind = OP_RELAYOUT_NHWC_TO_44;
        return true;
    }
    if (sym.compare(0, 30, "cuda_sm100_relayout_NHWC_NCHW_") == 0) {
        op->kind = ends_with(sym, "f32f32") ? OP_RELAYOUT_F32_TO_NCHW : OP_RELAYOUT_TO_NCHW;
        return true;
    }
    return false;
}

size_t nr_elems(const Tensor* t) {
    size_t n = 1;
    for (int i = 0; i < t->layout.nr_dim; ++i)
        n *= t->layout.dims[i];
    return n;
}

void fill_conv_param(const OpPlan& op, Tensor* const* inputs, const Tensor* dst,
                     mb200_conv_param* p) {
    const Tensor* src = inputs[0];
    const Tensor* flt = inputs[1];
    memset(p, 0, sizeof(*p));
    p->n = src->layout.dims[0];
    p->ic = src->layout.dims[1];
    p->ih = src->layout.dims[2];
    p->iw = src->layout.dims[3];
    p->kh = op.kh;
    p->kw = op.kw;
    p->stride_h = op.sh;
    p->stride_w = op.sw;
    p->pad_h = op.ph;
    p->pad_w = op.pw;
    p->dilate_h = op.dh;
    p->dilate_w = op.dw;
    // the original filter is [OC][IC][KH][KW] or [G][OCpg][ICpg][KH][KW]; in the NCHW44
    // layouts the leading extent counts blocks of four output channels (or groups)
    const Layout& l = flt->layout;
    if (op.flt44) {
        // (after Init the first-layer filter may be a flat buffer: with dst given, the
        // channel count comes from dst)
        p->groups = op.dense ? 1 : (int)l.dims[0] * 4;
        p->oc = dst ? (int)dst->layout.dims[1] : (int)l.dims[0] * 4;
    } else {
        p->groups = op.dense ? 1 : (int)l.dims[0];
        p->oc = dst ? (int)dst->layout.dims[1]
                    : (op.dense ? (int)l.dims[0] : (int)(l.dims[0] * l.dims[1]));
    }
    p->nonline = op.mode;
    p->src_scale = src->dtype.param.scale;
    p->flt_scale = flt->dtype.param.scale;
    p->dst_scale = dst ? dst->dtype.param.scale : 1.f;
}

void fill_conv_f32_param(const OpPlan& op, Tensor* const* inputs, mb200_conv_f32_param* p) {
    const Tensor* src = inputs[0];
    const Layout& l = inputs[1]->layout;
    memset(p, 0, sizeof(*p));
    p->n = src->layout.dims[0];
    p->ic = src->layout.dims[1];
    p->ih = src->layout.dims[2];
    p->iw = src->layout.dims[3];
    p->oc = op.oc;
    p->kh = op.kh;
    p->kw = op.kw;
    p->stride_h = op.sh;
    p->stride_w = op.sw;
    p->pad_h = op.ph;
    p->pad_w = op.pw;
    // the processed filter is a flat buffer: a grouped filter's channels per group are part
    // of the symbol
    (void)l;
    p->groups = op.dense || op.icpg <= 0 ? 1 : p->ic / op.icpg;
    p->nonline = op.mode;
}

int matrix_k(const Tensor* a) {
    return (int)(nr_elems(a) / (size_t)a->layout.dims[0]);
}

// The library's own KernelFunc: what the generated stub of op.symbol does
// (megcc_b200/compiler/cuda_kernel_pack.cpp). One function serves every symbol; the
// attributes a stub has baked in come from the Opr's parsed symbol, which the VM passes in
// RuntimeOpt::opr.
TinyNNStatus builtin_kernel(
        Tensor** inputs, int nr_input, Tensor** outputs, int nr_output, const Workspace* ws,
        const RuntimeOpt* opt) {
    if (!opt || !opt->opr || nr_input < 1 || nr_output < 1)
        return TinyNN_ERROR_NULL_PTR;
    const OpPlan& op = *(const OpPlan*)opt->opr;
    void* st = opt->stream;
    Tensor* dst = outputs[0];
    switch (op.kind) {
        case OP_CONV: {
            mb200_conv_param p;
            fill_conv_param(op, inputs, dst, &p);
            const Tensor* src = inputs[0];
            // inputs: src, filter, [bias], [channel scales], [z, mid scale]
            const int scale_idx = op.has_bias ? 3 : 2;
            const int nr_plain = nr_input - (op.z_mode ? 2 : 0);
            const int32_t* bias = op.has_bias ? (const int32_t*)inputs[2]->ptr : nullptr;
            const float* ch = nr_plain > scale_idx ? (const float*)inputs[scale_idx]->ptr : nullptr;
            if (op.z_mode) {
                const Tensor* z = inputs[nr_input - 2];
                mb200_conv_fuse fuse;
                fuse.z = (const int8_t*)z->ptr;
                fuse.mode = op.z_mode - 1;
                fuse.z_scale = z->dtype.param.scale;
                fuse.out_scale = dst->dtype.param.scale;
                p.dst_scale = inputs[nr_input - 1]->dtype.param.scale;  // scale of the ConvBias result
                return (TinyNNStatus)mb200_conv_bias_qs8_nhwc_fused(
                        &p, (const int8_t*)src->ptr, src->layout.format == TinyNN_NCHW,
                        (const int8_t*)inputs[1]->ptr, bias, ch, &fuse, (int8_t*)dst->ptr,
                        MB200_ALGO_AUTO, st);
            }
            if (op.pool)
                return (TinyNNStatus)mb200_conv_bias_pool_qs8_s2d(
                        &p, (const int8_t*)src->ptr, src->layout.format == TinyNN_NCHW,
                        (const int8_t*)inputs[1]->ptr, bias, ch, (int8_t*)dst->ptr, ws->ptr,
                        ws->size, st);
            if (mb200_conv_s2d_supported(&p))
                return (TinyNNStatus)mb200_conv_bias_qs8_s2d(
                        &p, (const int8_t*)src->ptr, src->layout.format == TinyNN_NCHW,
                        (const int8_t*)inputs[1]->ptr, bias, ch, (int8_t*)dst->ptr, ws->ptr,
                        ws->size, st);
            return (TinyNNStatus)mb200_conv_bias_qs8_nhwc(
                    &p, (const int8_t*)src->ptr, src->layout.format == TinyNN_NCHW,
                    (const int8_t*)inputs[1]->ptr, bias, ch, (int8_t*)dst->ptr, MB200_ALGO_AUTO, st);
        }
        case OP_POOL: {
            const Tensor* s = inputs[0];
            return (TinyNNStatus)mb200_pooling_qs8_nhwc(
                    (const int8_t*)s->ptr, (int8_t*)dst->ptr, op.mode, s->layout.dims[0],
                    s->layout.dims[1], s->layout.dims[2], s->layout.dims[3], op.kh, op.kw, op.sh,
                    op.sw, op.ph, op.pw, st);
        }
        case OP_QELEM: {
            const Tensor* a = inputs[0];
            const Tensor* b = nr_input > 1 ? inputs[1] : inputs[0];
            return (TinyNNStatus)mb200_qelemwise_qs8(
                    (const int8_t*)a->ptr, (const int8_t*)b->ptr, (int8_t*)dst->ptr, op.mode,
                    nr_elems(a), a->dtype.param.scale, b->dtype.param.scale,
                    dst->dtype.param.scale, st);
        }
        case OP_MATMUL: {
            const Tensor* a = inputs[0];
            const Tensor* b = inputs[1];  // re-laid to [N][K] at load
            // scale of the qint32 product: one float multiplication, as MegEngine records it
            const float acc_scale = a->dtype.param.scale * b->dtype.param.scale;
            return (TinyNNStatus)mb200_matmul_s8_qs8(
                    a->layout.dims[0], dst->layout.dims[1], matrix_k(a), (const int8_t*)a->ptr,
                    (const int8_t*)b->ptr, (int8_t*)dst->ptr, acc_scale, dst->dtype.param.scale, st);
        }
        case OP_TYPECVT: {
            const Tensor* s = inputs[0];
            return (TinyNNStatus)mb200_typecvt_qs32_qs8(
                    (const int32_t*)s->ptr, (int8_t*)dst->ptr, nr_elems(s), s->dtype.param.scale,
                    dst->dtype.param.scale, st);
        }
        case OP_RELAYOUT_TO_NHWC:
        case OP_RELAYOUT_TO_NCHW: {
            const Tensor* s = inputs[0];
            auto fn = op.kind == OP_RELAYOUT_TO_NHWC ? mb200_relayout_nchw_to_nhwc_s8
                                                     : mb200_relayout_nhwc_to_nchw_s8;
            return (TinyNNStatus)fn((const int8_t*)s->ptr, (int8_t*)dst->ptr, s->layout.dims[0],
                                    s->layout.dims[1], s->layout.dims[2], s->layout.dims[3], st);
        }
        case OP_RELAYOUT_44_TO_NHWC: {  // src [N][C/4][H][W][4]
            const Tensor* s = inputs[0];
            return (TinyNNStatus)mb200_relayout_nchw44_to_nhwc_s8(
                    (const int8_t*)s->ptr, (int8_t*)dst->ptr, s->layout.dims[0],
                    s->layout.dims[1] * 4, s->layout.dims[2], s->layout.dims[3], st);
        }
        case OP_RELAYOUT_NHWC_TO_44: {
            const Tensor* s = inputs[0];
            return (TinyNNStatus)mb200_relayout_nhwc_to_nchw44_s8(
                    (const int8_t*)s->ptr, (int8_t*)dst->ptr, s->layout.dims[0], s->layout.dims[1],
                    s->layout.dims[2], s->layout.dims[3], st);
        }
        case OP_RELAYOUT_F32_TO_NHWC:
        case OP_RELAYOUT_F32_TO_NCHW: {
            const Tensor* s = inputs[0];
            auto fn = op.kind == OP_RELAYOUT_F32_TO_NHWC ? mb200_relayout_nchw_to_nhwc_f32
                                                         : mb200_relayout_nhwc_to_nchw_f32;
            return (TinyNNStatus)fn((const float*)s->ptr, (float*)dst->ptr, s->layout.dims[0],
                                    s->layout.dims[1], s->layout.dims[2], s->layout.dims[3], st);
        }
        case OP_CONV_F32: {
            mb200_conv_f32_param p;
            fill_conv_f32_param(op, inputs, &p);
            const float* bias = op.has_bias ? (const float*)inputs[2]->ptr : nullptr;
            const float* z = op.f32_z ? (const float*)inputs[nr_input - 1]->ptr : nullptr;
            return (TinyNNStatus)mb200_conv_bias_f32_nhwc(
                    &p, (const float*)inputs[0]->ptr, (const float*)inputs[1]->ptr, bias, z,
                    (float*)dst->ptr, (long long)dst->layout.stride[3], ws->ptr, ws->size,
                    MB200_ALGO_AUTO, st);
        }
        case OP_MATMUL_F32: {
            const Tensor* a = inputs[0];
            return (TinyNNStatus)mb200_matmul_f32(
                    a->layout.dims[0], dst->layout.dims[1], matrix_k(a), (const float*)a->ptr,
                    (const float*)inputs[1]->ptr, (float*)dst->ptr, ws->ptr, ws->size, st);
        }
        case OP_ELEM_F32: {
            const Tensor* a = inputs[0];
            const Tensor* b = nr_input > 1 ? inputs[1] : inputs[0];
            return (TinyNNStatus)mb200_elemwise_f32(op.mode, (const float*)a->ptr,
                                                    (const float*)b->ptr, (float*)dst->ptr,
                                                    nr_elems(a), st);
        }
        case OP_CONCAT_F32: {
            const float* srcs[8];
            int channels[8];
            if (nr_input > 8)
                return TinyNN_ERROR_OUT_OF_RANGE;
            for (int i = 0; i < nr_input; ++i) {
                srcs[i] = (const float*)inputs[i]->ptr;
                channels[i] = inputs[i]->layout.dims[1];
            }
            return (TinyNNStatus)mb200_concat_f32_nhwc(
                    srcs, channels, nr_input, (float*)dst->ptr,
                    (size_t)dst->layout.dims[0] * dst->layout.dims[2] * dst->layout.dims[3], st);
        }
        case OP_FOCUS_F32: {
            const Tensor* s = inputs[0];
            return (TinyNNStatus)mb200_focus_f32(
                    (const float*)s->ptr, (float*)dst->ptr, s->layout.dims[0], s->layout.dims[1],
                    s->layout.dims[2], s->layout.dims[3], dst->layout.dims[1], st);
        }
        case OP_RESIZE_F32: {
            const Tensor* s = inputs[0];
            return (TinyNNStatus)mb200_resize_nearest_f32_nhwc(
                    (const float*)s->ptr, (float*)dst->ptr, s->layout.dims[0], s->layout.dims[1],
                    s->layout.dims[2], s->layout.dims[3], dst->layout.dims[2], dst->layout.dims[3],
                    st);
        }
        case OP_POOL_F32: {
            const Tensor* s = inputs[0];
            return (TinyNNStatus)mb200_pooling_f32_nhwc(
                    (const float*)s->ptr, (float*)dst->ptr, op.mode, s->layout.dims[0],
                    s->layout.dims[1], s->layout.dims[2], s->layout.dims[3], op.kh, op.kw, op.sh,
                    op.sw, op.ph, op.pw, st);
        }
        case OP_EXTERNAL:
            break;
    }
    return TinyNN_ERROR_NO_IMPLEMENT;
}

// The library's own InitFunc, in the three-phase protocol of runtime/src/data_struct.h
// :135-142 (count -> describe -> fill): ConvBias filters are re-laid K-major (or into the
// space-to-depth / tf32-plane forms), MatrixMul's B is transposed.
TinyNNStatus builtin_init(
        Tensor** inputs, int nr_input, Tensor* out_weights, int* nr_out_weight,
        const RuntimeOpt* opt) {
    if (!opt || !opt->opr || nr_input < 2)
        return TinyNN_ERROR_NULL_PTR;
    const OpPlan& op = *(const OpPlan*)opt->opr;
    if (!op.needs_init) {
        if (nr_out_weight)
            *nr_out_weight = 0;
        return TinyNN_SUCCESS;
    }
    if (!out_weights && nr_out_weight) {
        *nr_out_weight = 1;
        return TinyNN_SUCCESS;
    }
    Tensor* w = inputs[1];
    const bool describe = out_weights && !nr_out_weight;
    auto flat = [&](size_t elems) {
        out_weights->layout.nr_dim = 1;
        out_weights->layout.dims[0] = (uint32_t)elems;
        out_weights->layout.stride[0] = 1;
        out_weights->layout.format = w->layout.format;
        out_weights->dtype = w->dtype;
        out_weights->name = w->name;
    };
    switch (op.kind) {
        case OP_CONV: {
            if (w->layout.nr_dim < 4 || w->layout.nr_dim > 6)
                return TinyNN_ERROR_INVALID_LAYOUT;
            mb200_conv_param p;
            fill_conv_param(op, inputs, nullptr, &p);
            const bool s2d = !op.z_mode && mb200_conv_s2d_supported(&p);
            if (describe) {
                // the K-major filter keeps the layout (the kernel reads the group count from
                // it); the space-to-depth packing is a flat byte buffer
                if (s2d) {
                    flat(mb200_conv_s2d_filter_bytes(&p));
                } else {
                    out_weights->layout = w->layout;
                    out_weights->dtype = w->dtype;
                    out_weights->name = w->name;
                }
                return TinyNN_SUCCESS;
            }
            if (op.flt44)
                return (TinyNNStatus)mb200_conv_pack_filter_nchw44(
                        &p, op.flt44 - 1, (const int8_t*)w->ptr, (int8_t*)out_weights->ptr,
                        opt->stream);
            return (TinyNNStatus)(
                    s2d ? mb200_conv_s2d_pack_filter(&p, (const int8_t*)w->ptr,
                                                     (int8_t*)out_weights->ptr, opt->stream)
                        : mb200_conv_pack_filter(&p, (const int8_t*)w->ptr,
                                                 (int8_t*)out_weights->ptr, opt->stream));
        }
        case OP_MATMUL: {
            if (w->layout.nr_dim != 2)
                return TinyNN_ERROR_INVALID_LAYOUT;
            const int k = w->layout.dims[0], n = w->layout.dims[1];
            if (describe) {
                flat((size_t)k * n);
                return TinyNN_SUCCESS;
            }
            return (TinyNNStatus)mb200_matmul_pack_b(k, n, (const int8_t*)w->ptr,
                                                     (int8_t*)out_weights->ptr, opt->stream);
        }
        case OP_CONV_F32: {
            if (w->layout.nr_dim != 4 && w->layout.nr_dim != 5)
                return TinyNN_ERROR_INVALID_LAYOUT;
            mb200_conv_f32_param p;
            fill_conv_f32_param(op, inputs, &p);
            if (describe) {
                flat(mb200_conv_f32_packed_filter_bytes(&p) / 4);
                return TinyNN_SUCCESS;
            }
            return (TinyNNStatus)mb200_conv_f32_pack_filter(
                    &p, (const float*)w->ptr, (float*)out_weights->ptr, opt->stream);
        }
        case OP_MATMUL_F32: {
            if (w->layout.nr_dim != 2)
                return TinyNN_ERROR_INVALID_LAYOUT;
            const int k = w->layout.dims[0], n = w->layout.dims[1];
            if (describe) {
                flat(mb200_matmul_f32_packed_b_bytes(k, n) / 4);
                return TinyNN_SUCCESS;
            }
            return (TinyNNStatus)mb200_matmul_f32_pack_b(k, n, (const float*)w->ptr,
                                                         (float*)out_weights->ptr, opt->stream);
        }
        default:
            break;
    }
    return TinyNN_ERROR_NO_IMPLEMENT;
}

// Operand ranks and extents of an instruction against what its kernel will compute, so that a
// truncated or hand-edited model cannot make a kernel read or write outside its tensors.
// Returns a description of the first inconsistency, or nullptr.
const char* check_operands(const OpPlan& op) {
    auto rank4 = [](const Tensor* t) { return t->layout.nr_dim == 4; };
    auto extent = [](int in, int k, int s, int p) { return (in + 2 * p - k) / s + 1; };
    const Tensor* in0 = op.inputs[0];
    const Tensor* out = op.outputs[0];
    switch (op.kind) {
        case OP_CONV:
        case OP_CONV_F32: {
            const Tensor* flt = op.inputs[1];
            if (!rank4(in0) || !rank4(out))
                return "ConvBias operands must have 4 dims";
            if (!flt->is_weight)
                return "ConvBias filter must be a weight";
            if (op.kh <= 0 || op.kw <= 0 || op.sh <= 0 || op.sw <= 0)
                return "ConvBias attributes";
            const Layout& l = flt->layout;
            size_t oc, icpg, groups;
            if (op.flt44 == 1) {
                // [OC/4][IC/4][KH][KW][4][4]
                if (l.nr_dim != 6 || l.dims[2] != (uint32_t)op.kh || l.dims[3] != (uint32_t)op.kw ||
                    l.dims[4] != 4 || l.dims[5] != 4 || !op.dense)
                    return "dense NCHW44 filter must be [OC/4][IC/4][KH][KW][4][4]";
                oc = (size_t)l.dims[0] * 4, icpg = (size_t)l.dims[1] * 4, groups = 1;
            } else if (op.flt44 == 2) {
                // [G/4][1][1][KH][KW][4]
                if (l.nr_dim != 6 || l.dims[1] != 1 || l.dims[2] != 1 ||
                    l.dims[3] != (uint32_t)op.kh || l.dims[4] != (uint32_t)op.kw ||
                    l.dims[5] != 4 || op.dense)
                    return "channel-wise NCHW44 filter must be [G/4][1][1][KH][KW][4]";
                oc = groups = (size_t)l.dims[0] * 4, icpg = 1;
            } else if (op.flt44 == 3) {
                // [OC/4][KH][KW][IC][4]
                if (l.nr_dim != 5 || l.dims[4] != 4 || l.dims[1] != (uint32_t)op.kh ||
                    l.dims[2] != (uint32_t)op.kw || !op.dense)
                    return "first-layer NCHW44 filter must be [OC/4][KH][KW][IC][4]";
                oc = (size_t)l.dims[0] * 4, icpg = l.dims[3], groups = 1;
            } else {
                if (l.nr_dim != 4 && l.nr_dim != 5)
                    return "ConvBias filter must have 4 or 5 dims";
                oc = l.nr_dim == 4 ? l.dims[0] : (size_t)l.dims[0] * l.dims[1];
                icpg = l.nr_dim == 4 ? l.dims[1] : l.dims[2];
                groups = l.nr_dim == 4 ? 1 : l.dims[0];
                if (l.dims[l.nr_dim - 2] != (uint32_t)op.kh ||
                    l.dims[l.nr_dim - 1] != (uint32_t)op.kw)
                    return "filter extent differs from the symbol";
                if (op.dense != (l.nr_dim == 4))
                    return "filter rank does not match the sparse mode";
            }
            if (icpg * groups != in0->layout.dims[1] || oc != out->layout.dims[1])
                return "filter channels do not match the tensors";
            int oh = extent(in0->layout.dims[2], op.kh, op.sh, op.ph);
            int ow = extent(in0->layout.dims[3], op.kw, op.sw, op.pw);
            if (op.pool) {  // MAX pooling 3x3 / 2 / pad 1 behind the ConvBias
                if (op.kind != OP_CONV || op.z_mode || oh < 1 || ow < 1)
                    return "ConvBias + pooling operands";
                oh = extent(oh, 3, 2, 1);
                ow = extent(ow, 3, 2, 1);
            }
            if (out->layout.dims[0] != in0->layout.dims[0] || (int)out->layout.dims[2] != oh ||
                (int)out->layout.dims[3] != ow)
                return "output extent differs from what the ConvBias computes";
            const size_t extra = op.inputs.size() - 2;
            size_t idx = 2;
            if (op.has_bias) {
                if (extra < 1 || nr_elems(op.inputs[2]) != oc || !op.inputs[2]->is_weight)
                    return "bias must be a weight with one value per output channel";
                ++idx;
            }
            if (op.kind == OP_CONV_F32) {
                if (op.oc != (int)oc)
                    return "output channels differ from the symbol";
                if (op.f32_z && (op.inputs.size() <= idx || op.inputs.back()->size != out->size))
                    return "z does not match the output";
            } else if (op.inputs.size() - (op.z_mode ? 2 : 0) > idx &&
                       nr_elems(op.inputs[idx]) != oc) {
                return "channel scales must hold one value per output channel";
            }
            return nullptr;
        }
        case OP_POOL:
        case OP_POOL_F32:
            if (!rank4(in0) || !rank4(out))
                return "Pooling operands must have 4 dims";
            if (op.kh <= 0 || op.kw <= 0 || op.sh <= 0 || op.sw <= 0 ||
                out->layout.dims[0] != in0->layout.dims[0] ||
                out->layout.dims[1] != in0->layout.dims[1] ||
                (int)out->layout.dims[2] != extent(in0->layout.dims[2], op.kh, op.sh, op.ph) ||
                (int)out->layout.dims[3] != extent(in0->layout.dims[3], op.kw, op.sw, op.pw))
                return "output extent differs from what the Pooling computes";
            return nullptr;
        case OP_MATMUL:
        case OP_MATMUL_F32: {
            const Tensor* b = op.inputs[1];
            if (!b->is_weight || b->layout.nr_dim != 2 || in0->layout.nr_dim < 2 ||
                out->layout.nr_dim < 2)
                return "MatrixMul operands";
            if (nr_elems(in0) != (size_t)in0->layout.dims[0] * b->layout.dims[0] ||
                nr_elems(out) != (size_t)in0->layout.dims[0] * b->layout.dims[1] ||
                out->layout.dims[0] != in0->layout.dims[0] || out->layout.dims[1] != b->layout.dims[1])
                return "MatrixMul extents do not match";
            return nullptr;
        }
        case OP_RELAYOUT_TO_NHWC:
        case OP_RELAYOUT_TO_NCHW:
        case OP_RELAYOUT_F32_TO_NHWC:
        case OP_RELAYOUT_F32_TO_NCHW:
            if (!rank4(in0) || !rank4(out) || in0->size != out->size)
                return "Relayout operands must be 4-dim tensors of one size";
            for (int d = 0; d < 4; ++d)
                if (in0->layout.dims[d] != out->layout.dims[d])
                    return "Relayout keeps the logical extents";
            return nullptr;
        case OP_RELAYOUT_44_TO_NHWC:
        case OP_RELAYOUT_NHWC_TO_44: {
            const Tensor* t44 = op.kind == OP_RELAYOUT_44_TO_NHWC ? in0 : out;
            const Tensor* t4 = op.kind == OP_RELAYOUT_44_TO_NHWC ? out : in0;
            if (t44->layout.nr_dim != 5 || t44->layout.dims[4] != 4 || !rank4(t4) ||
                t44->layout.dims[0] != t4->layout.dims[0] ||
                t44->layout.dims[1] * 4 != t4->layout.dims[1] ||
                t44->layout.dims[2] != t4->layout.dims[2] ||
                t44->layout.dims[3] != t4->layout.dims[3])
                return "NCHW44 Relayout operands must be [N][C/4][H][W][4] and [N][C][H][W]";
            return nullptr;
        }
        case OP_QELEM:
        case OP_ELEM_F32:
            for (auto* t : op.inputs)
                if (t->size != out->size)
                    return "elementwise operands must have the output's size";
            return nullptr;
        case OP_TYPECVT:
            return nr_elems(in0) == nr_elems(out) ? nullptr : "TypeCvt element counts differ";
        case OP_CONCAT_F32: {
            if (!rank4(out) || op.inputs.size() > 8)
                return "Concat takes up to 8 inputs and a 4-dim output";
            size_t c = 0;
            for (auto* t : op.inputs) {
                if (!rank4(t) || t->layout.dims[0] != out->layout.dims[0] ||
                    t->layout.dims[2] != out->layout.dims[2] ||
                    t->layout.dims[3] != out->layout.dims[3])
                    return "Concat inputs must share the output's batch and spatial extents";
                c += t->layout.dims[1];
            }
            return c == out->layout.dims[1] ? nullptr : "Concat channel counts do not add up";
        }
        case OP_FOCUS_F32:
            if (!rank4(in0) || !rank4(out) || (in0->layout.dims[2] & 1) ||
                (in0->layout.dims[3] & 1) || out->layout.dims[0] != in0->layout.dims[0] ||
                out->layout.dims[1] < 4 * in0->layout.dims[1] ||
                out->layout.dims[2] * 2 != in0->layout.dims[2] ||
                out->layout.dims[3] * 2 != in0->layout.dims[3])
                return "Focus extents do not match";
            return nullptr;
        case OP_RESIZE_F32:
            if (!rank4(in0) || !rank4(out) || out->layout.dims[0] != in0->layout.dims[0] ||
                out->layout.dims[1] != in0->layout.dims[1])
                return "Resize keeps batch and channels";
            return nullptr;
        case OP_EXTERNAL:
            return nullptr;
    }
    return nullptr;
}

// ---------------------------------------------------------------------------------------
// model parsing
// ---------------------------------------------------------------------------------------
bool read_dtype(const fb::Table& t, DType* out) {
    if (!t)
        return false;
    out->type_enum = (TinyNNDType)(int)t.scalar<int8_t>(fb::field::DT_type, 0);
    const fb::Table p = t.table(fb::field::DT_param);
    out->param.scale = p ? p.scalar<float>(fb::field::DP_scale, 1.0f) : 1.0f;
    out->param.zero_point = p ? p.scalar<uint8_t>(fb::field::DP_zero_point, 0) : 0;
    switch (out->type_enum) {
        case TinyNN_FLOAT: case TinyNN_FLOAT16: case TinyNN_INT: case TinyNN_INT8:
        case TinyNN_INT16: case TinyNN_UINT8: case TinyNN_QINT8: case TinyNN_QINT32:
        case TinyNN_QUINT8:
            return true;
        default:
            return false;
    }
}

bool read_layout(const fb::Table& t, Layout* out) {
    if (!t)
        return false;
    const fb::Vec dims = t.vec(fb::field::L_dims, 4), stride = t.vec(fb::field::L_stride, 4);
    if (!dims || !stride || dims.len != stride.len || dims.len > MAX_DIM)
        return false;
    memset(out, 0, sizeof(*out));
    out->nr_dim = (int)dims.len;
    for (uint32_t i = 0; i < dims.len; ++i) {
        const int d = dims.at<int32_t>(i);
        if (d < 0)
            return false;
        out->dims[i] = (uint32_t)d;
        out->stride[i] = stride.at<int32_t>(i);
    }
    out->format = (TinyNNFormat)(int)t.scalar<int8_t>(fb::field::L_format, 0);
    return true;
}

int parse_model(Network* net, const void* mem, size_t size) {
    fb::Buffer buf;  // Tables keep a pointer to it; none outlives this call
    buf.data = (const uint8_t*)mem;
    buf.size = size;
    buf.failed = false;
    const fb::Table model = fb::root(buf);
    if (!model)
        return fail(TinyNN_ERROR_MODEL_PARSE, "model buffer of %zu bytes has no root table", size);
    const fb::Vec wpool = model.vec(fb::field::M_weight_pool, 4);
    const fb::Vec dmodels = model.vec(fb::field::M_device_models, 4);
    if (!wpool || !dmodels)
        return fail(TinyNN_ERROR_MODEL_PARSE, "model lacks weight_pool or device_models");

    // ---- weights (host view; uploaded later) ----
    net->weights.resize(wpool.len);
    net->weight_names.resize(wpool.len);
    net->weight_host.assign(wpool.len, nullptr);
    std::vector<const uint8_t*>& host_data = net->weight_host;
    for (uint32_t i = 0; i < wpool.len; ++i) {
        const fb::Table w = fb::Table::elem(wpool, i);
        Tensor& t = net->weights[i];
        memset(&t, 0, sizeof(t));
        if (!w || !read_dtype(w.table(fb::field::W_dtype), &t.dtype) ||
            !read_layout(w.table(fb::field::W_layout), &t.layout))
            return fail(TinyNN_ERROR_MODEL_PARSE, "weight %u is malformed", i);
        if (w.scalar<uint8_t>(fb::field::W_compressed, 0))
            return fail(TinyNN_ERROR_NO_IMPLEMENT, "compressed weights are not supported");
        const fb::Vec data = w.vec(fb::field::W_data, 1);
        t.size = tensor_bytes(t);
        if (t.size == SIZE_MAX)
            return fail(TinyNN_ERROR_MODEL_PARSE, "weight %u: extents overflow", i);
        if (!data || data.len != t.size)
            return fail(TinyNN_ERROR_MODEL_PARSE, "weight %u: %u data bytes for a %zu byte layout",
                        i, data ? data.len : 0, t.size);
        host_data[i] = data.bytes();
        if (!w.str(fb::field::W_name, &net->weight_names[i]))
            net->weight_names[i] = "weight:" + std::to_string(i);
        t.use_count = w.scalar<int32_t>(fb::field::W_use_count, 0);
        t.checksum = w.scalar<uint32_t>(fb::field::W_checksum, 0);
        t.is_weight = 1;
    }
    for (size_t i = 0; i < net->weights.size(); ++i)
        net->weights[i].name = (char*)net->weight_names[i].c_str();

    // ---- device models: keep the ones for this device (parse.c:404-421 keeps those that
    // pass valid_device_check) ----
    for (uint32_t mi = 0; mi < dmodels.len; ++mi) {
        const fb::Table dm = fb::Table::elem(dmodels, mi);
        if (!dm)
            return fail(TinyNN_ERROR_MODEL_PARSE, "device model %u is malformed", mi);
        if (dm.scalar<int8_t>(fb::field::D_device, 0) != fb::CUDA_SM100)
            continue;
        net->models.emplace_back();
        DevModel& m = net->models.back();
        const fb::Vec tpool = dm.vec(fb::field::D_tensor_pool, 4);
        if (!tpool)
            return fail(TinyNN_ERROR_MODEL_PARSE, "device model %u has no tensor_pool", mi);
        m.tensors.resize(tpool.len);
        m.names.resize(tpool.len);
        m.tensor_memory = (size_t)dm.scalar<uint64_t>(fb::field::D_tensor_memory, 0);
        for (uint32_t i = 0; i < tpool.len; ++i) {
            const fb::Table tt = fb::Table::elem(tpool, i);
            Tensor& t = m.tensors[i];
            memset(&t, 0, sizeof(t));
            if (!tt || !read_dtype(tt.table(fb::field::T_dtype), &t.dtype) ||
                !read_layout(tt.table(fb::field::T_layout), &t.layout))
                return fail(TinyNN_ERROR_MODEL_PARSE, "tensor %u is malformed", i);
            if (tt.scalar<uint8_t>(fb::field::T_dynamic, 0))
                return fail(TinyNN_ERROR_NO_IMPLEMENT, "dynamic-shape tensors are not supported");
            const int64_t off = tt.scalar<int64_t>(fb::field::T_offset, 0);
            t.size = tensor_bytes(t);
            if (t.size == SIZE_MAX)
                return fail(TinyNN_ERROR_MODEL_PARSE, "tensor %u: extents overflow", i);
            if (off < 0 || (size_t)off > m.tensor_memory || t.size > m.tensor_memory - (size_t)off)
                return fail(TinyNN_ERROR_MODEL_PARSE,
                            "tensor %u at offset %lld (+%zu) lies outside the %zu byte arena", i,
                            (long long)off, t.size, m.tensor_memory);
            t.offset = (size_t)off;
            t.use_count = tt.scalar<int32_t>(fb::field::T_use_count, 0);
            if (!tt.str(fb::field::T_name, &m.names[i]) || m.names[i].empty())
                m.names[i] = "tensor:" + std::to_string(i);
        }
        for (size_t i = 0; i < m.tensors.size(); ++i)
            m.tensors[i].name = (char*)m.names[i].c_str();

        auto io = [&](int fid, std::vector<IoSlot>* slots, bool input) -> bool {
            const fb::Vec v = dm.vec(fid, 4);
            if (!v)
                return false;
            for (uint32_t i = 0; i < v.len; ++i) {
                const int idx = v.at<int32_t>(i);
                if (idx < 0 || (size_t)idx >= m.tensors.size())
                    return false;
                IoSlot s;
                s.tensor = &m.tensors[idx];
                s.bytes = s.tensor->size;
                if (input)
                    s.tensor->is_input = 1;
                for (auto& n : net->io_device_names)
                    if (n == s.tensor->name)
                        s.want_device = true;
                slots->push_back(s);
            }
            return true;
        };
        if (!io(fb::field::D_inputs, &m.inputs, true) || !io(fb::field::D_outputs, &m.outputs, false))
            return fail(TinyNN_ERROR_MODEL_PARSE, "device model %u: bad input/output index", mi);

        const fb::Vec itypes = dm.vec(fb::field::D_instructions_type, 1);
        const fb::Vec insts = dm.vec(fb::field::D_instructions, 4);
        if (!itypes || !insts || itypes.len != insts.len)
            return fail(TinyNN_ERROR_MODEL_PARSE, "device model %u: instruction vectors differ", mi);
        m.instrs.reserve(insts.len);
        for (uint32_t i = 0; i < insts.len; ++i) {
            const uint8_t tag = itypes.at<uint8_t>(i);
            const fb::Table it = fb::Table::elem(insts, i);
            if (!it)
                return fail(TinyNN_ERROR_MODEL_PARSE, "instruction %u is malformed", i);
            Instr ins;
            if (tag == fb::INST_OPR) {
                ins.is_opr = true;
                std::string type;
                if (!it.str(fb::field::O_type, &type))
                    return fail(TinyNN_ERROR_MODEL_PARSE, "instruction %u has no type", i);
                // Dispatch goes through the function tables by kernel_id / init_id
                // (runtime/src/vm/op.c:161-163): a registered table entry wins, else the
                // library's own implementation of the symbol fills the slot.
                const bool known = parse_symbol(type, &ins.op);
                ins.op.kernel_id = it.scalar<int32_t>(fb::field::O_kernel_id, -1);
                ins.op.init_id = it.scalar<int32_t>(fb::field::O_init_id, -1);
                KernelFunc ext = ins.op.kernel_id >= 0 &&
                                                 (size_t)ins.op.kernel_id < net->ext_kernels.size()
                                         ? net->ext_kernels[ins.op.kernel_id]
                                         : nullptr;
                if (ext) {
                    ins.op.kernel_fn = ext;
                    ins.op.init_fn = ins.op.init_id >= 0 &&
                                                     (size_t)ins.op.init_id < net->ext_inits.size()
                                             ? net->ext_inits[ins.op.init_id]
                                             : nullptr;
                    if (!known) {
                        ins.op.kind = OP_EXTERNAL;
                        ins.op.symbol = type;
                    }
                } else if (known) {
                    ins.op.kernel_fn = builtin_kernel;
                    ins.op.init_fn = ins.op.needs_init ? builtin_init : nullptr;
                } else {
                    return fail(TinyNN_ERROR_NO_FOUND,
                                "instruction %u: no sm_100a kernel for symbol '%s' and no "
                                "registered kernel table entry %d", i, type.c_str(),
                                ins.op.kernel_id);
                }
                it.str(fb::field::O_name, &ins.op.name);
                const fb::Vec in = it.vec(fb::field::O_inputs, 4);
                const fb::Vec in_t = it.vec(fb::field::O_input_types, 1);
                const fb::Vec out = it.vec(fb::field::O_outputs, 4);
                if (!in || !in_t || !out || in.len != in_t.len)
                    return fail(TinyNN_ERROR_MODEL_PARSE, "instruction %u: operand lists", i);
                for (uint32_t k = 0; k < in.len; ++k) {
                    const int idx = in.at<int32_t>(k);
                    const bool is_w = in_t.at<int8_t>(k) == fb::WEIGHT;
                    const size_t limit = is_w ? net->weights.size() : m.tensors.size();
                    if (idx < 0 || (size_t)idx >= limit)
                        return fail(TinyNN_ERROR_MODEL_PARSE, "instruction %u: operand %u", i, k);
                    if (is_w)
                        ins.op.weight_inputs.push_back((int)k);
                    ins.op.inputs.push_back(is_w ? &net->weights[idx] : &m.tensors[idx]);
                }
                for (uint32_t k = 0; k < out.len; ++k) {
                    const int idx = out.at<int32_t>(k);
                    if (idx < 0 || (size_t)idx >= m.tensors.size())
                        return fail(TinyNN_ERROR_MODEL_PARSE, "instruction %u: output %u", i, k);
                    ins.op.outputs.push_back(&m.tensors[idx]);
                }
                // the workspace table is always present (runtime/src/vm/op.c:56-58)
                const fb::Table ws = it.table(fb::field::O_workspace);
                if (!ws)
                    return fail(TinyNN_ERROR_MODEL_PARSE, "instruction %u: no workspace", i);
                ins.op.ws.size = (size_t)ws.scalar<int64_t>(fb::field::WS_size, 0);
                ins.op.ws.offset = (size_t)ws.scalar<int64_t>(fb::field::WS_offset, 0);
                if (ins.op.ws.size && ins.op.ws.offset + ins.op.ws.size > m.tensor_memory)
                    return fail(TinyNN_ERROR_MODEL_PARSE, "instruction %u: workspace outside arena",
                                i);
                const size_t need_in = (ins.op.kind == OP_CONV || ins.op.kind == OP_CONV_F32 ||
                                        ins.op.kind == OP_MATMUL || ins.op.kind == OP_MATMUL_F32)
                                               ? 2
                                               : 1;
                if (ins.op.inputs.size() < need_in || ins.op.outputs.empty())
                    return fail(TinyNN_ERROR_MODEL_PARSE, "instruction %u: too few operands", i);
                if (const char* why = check_operands(ins.op))
                    return fail(TinyNN_ERROR_MODEL_PARSE, "instruction %u (%s): %s", i,
                                type.c_str(), why);
                if (ins.op.kind == OP_CONV &&
                    ins.op.inputs.size() < (size_t)(ins.op.has_bias ? 3 : 2) + (ins.op.z_mode ? 2 : 0))
                    return fail(TinyNN_ERROR_MODEL_PARSE, "instruction %u: conv operand missing", i);
                if (ins.op.kind == OP_CONV && ins.op.z_mode) {
                    const Tensor* z = ins.op.inputs[ins.op.inputs.size() - 2];
                    const Tensor* o = ins.op.outputs[0];
                    if (z->is_weight || z->size != o->size || !ins.op.inputs.back()->is_weight)
                        return fail(TinyNN_ERROR_MODEL_PARSE,
                                    "instruction %u: fused operand does not match the output", i);
                }
            } else if (tag == fb::INST_MEM_FORWARD) {
                ins.is_opr = false;
                const int a = it.scalar<int32_t>(fb::field::MF_input, 0);
                const int b = it.scalar<int32_t>(fb::field::MF_output, 0);
                if (a < 0 || b < 0 || (size_t)a >= m.tensors.size() || (size_t)b >= m.tensors.size())
                    return fail(TinyNN_ERROR_MODEL_PARSE, "instruction %u: memforward index", i);
                ins.mf = {&m.tensors[a], &m.tensors[b], it.scalar<int32_t>(fb::field::MF_offset, 0)};
            } else {
                return fail(TinyNN_ERROR_UNSUPPORTED_INSTRUCTION_TYPE,
                            "instruction %u: type %u is not supported on the CUDA device", i,
                            (unsigned)tag);
            }
            m.instrs.push_back(std::move(ins));
        }
        if (m.tensor_memory > net->arena_need)
            net->arena_need = m.tensor_memory;
    }
    if (buf.failed)
        return fail(TinyNN_ERROR_MODEL_PARSE, "model buffer is truncated or corrupt");
    if (net->models.empty())
        return fail(TinyNN_ERROR_NO_FOUND, "model holds no DeviceModel for CUDA_SM100");

    return TinyNN_SUCCESS;
}

// weights -> one device allocation, then the Init step of every Opr that has one, through
// its InitFunc in the reference's three-phase protocol (runtime/src/init.c:29-131):
//   init(inputs, n, NULL, &count)   how many processed weights (at most one)
//   init(inputs, n, &w, NULL)       layout / dtype / name of the processed weight
//   init(inputs, n, &w, &count)     fill w.ptr (device memory here)
// after which the Opr's input whose name pointer equals the processed weight's is swapped for
// it (runtime/src/init.c:59-92). Oprs that preprocess the same weight in the same way share
// the result.
int upload_weights(Network* net) {
    std::vector<const uint8_t*>& host_data = net->weight_host;
    cudaError_t e = cudaSetDevice(net->device_id);
    if (e != cudaSuccess)
        return cuda_fail(e, "cudaSetDevice");
    if (!net->stream && (e = cudaStreamCreateWithFlags(&net->stream, cudaStreamNonBlocking)) != cudaSuccess)
        return cuda_fail(e, "cudaStreamCreate");
    net->opt.device = &net->device;
    net->opt.stream = net->stream;
    net->opt.device_id = net->device_id;
    net->opt.opr = nullptr;

    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    size_t total = 0;
    for (auto& w : net->weights)
        total += up(w.size);

    struct Job {
        OpPlan* op;
        int input;      // which input the processed weight replaces
        int processed;  // index into net->processed
        bool fill;      // this job runs phase three (the others reuse its result)
    };
    std::vector<Job> jobs;
    struct Key {
        const Tensor* weight;
        void* fn;
        std::string symbol;
        size_t bytes;
        bool operator==(const Key& o) const {
            return weight == o.weight && fn == o.fn && symbol == o.symbol && bytes == o.bytes;
        }
    };
    std::vector<std::pair<Key, int>> seen;
    std::vector<Tensor> described;
    for (auto& m : net->models)
        for (auto& ins : m.instrs) {
            if (!ins.is_opr || !ins.op.init_fn)
                continue;
            OpPlan& op = ins.op;
            RuntimeOpt opt = net->opt;
            opt.opr = &op;
            int count = 0;
            int rc = op.init_fn(op.inputs.data(), (int)op.inputs.size(), nullptr, &count, &opt);
            if (rc)
                return fail(rc, "init of %s: %s", op.symbol.c_str(), mb200_last_error());
            if (count == 0)
                continue;
            if (count != 1)
                return fail(TinyNN_ERROR_NO_IMPLEMENT,
                            "init of %s wants %d processed weights; one is supported",
                            op.symbol.c_str(), count);
            Tensor w;
            memset(&w, 0, sizeof(w));
            rc = op.init_fn(op.inputs.data(), (int)op.inputs.size(), &w, nullptr, &opt);
            if (rc)
                return fail(rc, "init of %s: %s", op.symbol.c_str(), mb200_last_error());
            int input = -1;
            for (size_t j = 0; j < op.inputs.size(); ++j)
                if (op.inputs[j]->is_weight && op.inputs[j]->name == w.name)
                    input = (int)j;
            if (input < 0)
                return fail(TinyNN_ERROR_NO_FOUND,
                            "init of %s names a processed weight that matches no input",
                            op.symbol.c_str());
            w.size = tensor_bytes(w);
            if (w.size == SIZE_MAX || w.size == 0)
                return fail(TinyNN_ERROR_INVALID_LAYOUT, "init of %s: bad processed layout",
                            op.symbol.c_str());
            w.is_weight = 1;
            const Key key{op.inputs[input], (void*)op.init_fn, op.symbol, w.size};
            int idx = -1;
            for (auto& sk : seen)
                if (sk.first == key)
                    idx = sk.second;
            const bool fresh = idx < 0;
            if (fresh) {
                idx = (int)described.size();
                described.push_back(w);
                seen.push_back({key, idx});
                total += up(w.size);
            }
            jobs.push_back({&op, input, idx, fresh});
        }
    net->processed = described;  // no growth from here on: jobs point into it

    if (total == 0)
        total = 256;
    if ((e = cudaMalloc(&net->weight_arena, total)) != cudaSuccess)
        return cuda_fail(e, "cudaMalloc(weights)");
    size_t off = 0;
    for (size_t i = 0; i < net->weights.size(); ++i) {
        Tensor& w = net->weights[i];
        w.ptr = (uint8_t*)net->weight_arena + off;
        off += up(w.size);
        if (w.size &&
            (e = cudaMemcpyAsync(w.ptr, host_data[i], w.size, cudaMemcpyHostToDevice, net->stream)) !=
                    cudaSuccess)
            return cuda_fail(e, "cudaMemcpy(weights)");
    }
    for (auto& pw : net->processed) {
        pw.ptr = (uint8_t*)net->weight_arena + off;
        off += up(pw.size);
    }
    // phase three with the original weights in place, then the swap
    for (auto& job : jobs) {
        if (!job.fill)
            continue;
        RuntimeOpt opt = net->opt;
        opt.opr = job.op;
        int count = 1;
        const int rc = job.op->init_fn(job.op->inputs.data(), (int)job.op->inputs.size(),
                                       &net->processed[job.processed], &count, &opt);
        if (rc)
            return fail(rc, "preprocessing weight '%s' for %s: %s",
                        job.op->inputs[job.input]->name, job.op->symbol.c_str(),
                        mb200_last_error());
    }
    for (auto& job : jobs)
        job.op->inputs[job.input] = &net->processed[job.processed];
    if ((e = cudaStreamSynchronize(net->stream)) != cudaSuccess)
        return cuda_fail(e, "weight upload");
    if (!mb200::device_status_word(net->stream))
        return fail(TinyNN_ERROR_MEMORY_MALLOC, "%s", mb200_last_error());
    net->loaded = true;
    return TinyNN_SUCCESS;
}

// ---------------------------------------------------------------------------------------
// memory + execution
// ---------------------------------------------------------------------------------------
int init_model_memory(Network* net) {
    DevModel& m = net->models[net->active];
    if (m.memory_ready)
        return TinyNN_SUCCESS;
    cudaError_t e = cudaSetDevice(net->device_id);
    if (e != cudaSuccess)
        return cuda_fail(e, "cudaSetDevice");
    Arena& a = *net->arena;
    if (a.bytes < net->arena_need)
        a.bytes = net->arena_need;
    if (!a.ptr) {
        // one allocation for every tensor and workspace of the model, with 128 KiB behind
        // the last tensor: the tensor-core ConvBias describes a small activation (batch 1 of a
        // late layer) to the TMA unit as 128 KiB starting at it, and the whole arena is
        // declared readable for that
        a.device = net->device_id;
        const size_t total = (a.bytes ? a.bytes : 256) + kArenaSlack;
        if ((e = cudaMalloc(&a.ptr, total)) != cudaSuccess)
            return cuda_fail(e, "cudaMalloc(arena)");
        if ((e = cudaMemset((uint8_t*)a.ptr + total - kArenaSlack, 0, kArenaSlack)) != cudaSuccess)
            return cuda_fail(e, "cudaMemset(arena slack)");
        mb200_register_readable_range(a.ptr, total);
    }
    for (auto& t : m.tensors)
        t.ptr = (uint8_t*)a.ptr + t.offset;
    for (auto& ins : m.instrs) {
        if (ins.is_opr)
            ins.op.ws.ptr = ins.op.ws.size ? (uint8_t*)a.ptr + ins.op.ws.offset : nullptr;
        else
            ins.mf.out->ptr = (uint8_t*)ins.mf.in->ptr + ins.mf.offset;
    }
    for (auto& o : m.outputs) {
        if (!o.host_stage && !o.want_device &&
            (e = cudaMallocHost(&o.host_stage, o.bytes ? o.bytes : 1)) != cudaSuccess)
            return cuda_fail(e, "cudaMallocHost(output)");
    }
    m.memory_ready = true;
    return TinyNN_SUCCESS;
}

int issue_instructions(Network* net, DevModel& m, bool timed) {
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    if (timed) {
        cudaEventCreate(&ev0);
        cudaEventCreate(&ev1);
    }
    for (auto& ins : m.instrs) {
        if (!ins.is_opr)
            continue;  // memforward is resolved when the arena is laid out
        if (timed)
            cudaEventRecord(ev0, net->stream);
        // kernels[opr->kernel_id](inputs, nr_input, outputs, nr_output, &workspace, &opt)
        RuntimeOpt opt = net->opt;
        opt.opr = &ins.op;
        const int rc = ins.op.kernel_fn(ins.op.inputs.data(), (int)ins.op.inputs.size(),
                                        ins.op.outputs.data(), (int)ins.op.outputs.size(),
                                        &ins.op.ws, &opt);
        if (rc)
            return fail(rc, "kernel %s: %s", ins.op.symbol.c_str(), mb200_last_error());
        if (timed) {
            cudaEventRecord(ev1, net->stream);
            cudaEventSynchronize(ev1);
            float ms = 0;
            cudaEventElapsedTime(&ms, ev0, ev1);
            ins.op.ms_total += ms;
            ins.op.ms_count++;
        }
    }
    if (timed) {
        cudaEventDestroy(ev0);
        cudaEventDestroy(ev1);
    }
    return TinyNN_SUCCESS;
}

int forward(Network* net) {
    if (!net->loaded)
        return fail(TinyNN_ERROR, "LITE_forward before a model was loaded");
    int rc = init_model_memory(net);
    if (rc)
        return rc;
    DevModel& m = net->models[net->active];
    cudaError_t e = cudaSetDevice(net->device_id);
    if (e != cudaSuccess)
        return cuda_fail(e, "cudaSetDevice");

    // inputs: device pointers are used in place, host pointers are copied in
    std::vector<void*> in_ptrs;
    for (auto& s : m.inputs) {
        if (!s.user_ptr)
            return fail(TinyNN_ERROR_NULL_PTR,
                        "input '%s' has no memory: call LITE_reset_tensor_memory first",
                        s.tensor->name);
        if (s.user_is_device) {
            s.tensor->ptr = s.user_ptr;
        } else {
            s.tensor->ptr = (uint8_t*)net->arena->ptr + s.tensor->offset;
            if ((e = copy_input(net, s.tensor->ptr, s.user_ptr, s.bytes)) != cudaSuccess)
                return cuda_fail(e, "cudaMemcpyAsync(input)");
        }
        in_ptrs.push_back(s.tensor->ptr);
    }

    ComputeLane* lane = net->profile ? nullptr : compute_lane(net->device_id);
    std::unique_lock<std::mutex> lane_lock;
    if (lane) {
        lane_lock = std::unique_lock<std::mutex>(lane->mu);
        if (!lane->done &&
            (e = cudaEventCreateWithFlags(&lane->done, cudaEventDisableTiming)) != cudaSuccess)
            return cuda_fail(e, "cudaEventCreate");
        if (lane->recorded &&
            (e = cudaStreamWaitEvent(net->stream, lane->done, 0)) != cudaSuccess)
            return cuda_fail(e, "cudaStreamWaitEvent");
    }
    if (net->profile || !net->use_graph) {
        if ((rc = issue_instructions(net, m, net->profile)))
            return rc;
    } else {
        if (!m.ran_eager) {
            // the first pass runs eagerly: it also performs one-time set-up that may not
            // happen under stream capture
            if ((rc = issue_instructions(net, m, false)))
                return rc;
            m.ran_eager = true;
        } else {
            size_t hit = m.graphs.size();
            for (size_t i = 0; i < m.graphs.size(); ++i)
                if (m.graphs[i].inputs == in_ptrs) {
                    hit = i;
                    break;
                }
            if (hit < m.graphs.size()) {
                if (hit != 0)
                    std::rotate(m.graphs.begin(), m.graphs.begin() + hit, m.graphs.begin() + hit + 1);
            } else {
                if (m.graphs.size() >= DevModel::kMaxGraphs) {  // drop the least recently used
                    cudaGraphExecDestroy(m.graphs.back().exec);
                    m.graphs.pop_back();
                }
                cudaGraph_t graph = nullptr;
                if ((e = cudaStreamBeginCapture(net->stream, cudaStreamCaptureModeThreadLocal)) !=
                    cudaSuccess)
                    return cuda_fail(e, "cudaStreamBeginCapture");
                rc = issue_instructions(net, m, false);
                e = cudaStreamEndCapture(net->stream, &graph);
                if (rc) {
                    if (graph)
                        cudaGraphDestroy(graph);
                    return rc;
                }
                if (e != cudaSuccess)
                    return cuda_fail(e, "cudaStreamEndCapture");
                cudaGraphExec_t exec = nullptr;
                e = cudaGraphInstantiate(&exec, graph, 0);
                cudaGraphDestroy(graph);
                if (e != cudaSuccess)
                    return cuda_fail(e, "cudaGraphInstantiate");
                m.graphs.insert(m.graphs.begin(), DevModel::CapturedGraph{in_ptrs, exec});
            }
            if ((e = cudaGraphLaunch(m.graphs.front().exec, net->stream)) != cudaSuccess)
                return cuda_fail(e, "cudaGraphLaunch");
        }
    }
    if (lane) {
        if ((e = cudaEventRecord(lane->done, net->stream)) != cudaSuccess)
            return cuda_fail(e, "cudaEventRecord");
        lane->recorded = true;
        lane_lock.unlock();
    }
    for (auto& o : m.outputs) {
        if (o.want_device)
            continue;
        if ((e = cudaMemcpyAsync(o.host_stage, o.tensor->ptr, o.bytes, cudaMemcpyDeviceToHost,
                                 net->stream)) != cudaSuccess)
            return cuda_fail(e, "cudaMemcpyAsync(output)");
    }
    net->pending = true;
    return TinyNN_SUCCESS;
}

int wait(Network* net) {
    if (!net->pending)
        return TinyNN_SUCCESS;
    net->pending = false;
    cudaSetDevice(net->device_id);
    int status = 0;
    const int rc = mb200_device_status(net->stream, &status);  // synchronises the stream
    if (rc)
        return fail(rc, "%s", mb200_last_error());
    if (status)
        return fail(TinyNN_ERROR_RUNTIME, "a kernel gave up on a bounded wait (code 0x%x)", status);
    return TinyNN_SUCCESS;
}

Network* as_net(LiteNetwork n) {
    return (Network*)n;
}
IoHandle* as_io(LiteTensor t) {
    return (IoHandle*)t;
}
IoSlot* slot_of(IoHandle* h) {
    DevModel& m = h->net->models[h->net->active];
    auto& v = h->is_input ? m.inputs : m.outputs;
    return (size_t)h->index < v.size() ? &v[h->index] : nullptr;
}

LiteConfig g_default_config = {
        0, -1, LITE_CPU, LITE_DEFAULT, nullptr,
        {0, 0, 0, 1, 0, 0, 0, 0, 0, 0, 2, 1, 0, 0, 0, 0, 0, 0, 0}};
LiteNetworkIO g_default_io = {nullptr, nullptr, 0, 0};

}  // namespace

// ---------------------------------------------------------------------------------------
// C API
// ---------------------------------------------------------------------------------------
extern "C" {

LiteConfig* default_config(void) {
    return &g_default_config;
}
LiteNetworkIO* default_network_io(void) {
    return &g_default_io;
}

const char* LITE_get_last_error(void) {
    return g_lite_err;
}

int LITE_set_log_level(LiteLogLevel level) {
    g_log_level = level;
    return 0;
}
int LITE_get_log_level(LiteLogLevel* level) {
    if (!level)
        return TinyNN_ERROR_NULL_PTR;
    *level = g_log_level;
    return 0;
}

// Parses a model exactly as LITE_load_model_from_mem does, without touching a GPU, and
// writes a one-line-per-item text summary. For tools and tests.
int mb200_tinynn_describe(const void* model_mem, size_t size, char* out, size_t cap) {
    if (!model_mem || !out || !cap)
        return fail(TinyNN_ERROR_NULL_PTR, "input pointer is NULL");
    Network net;
    const int rc = parse_model(&net, model_mem, size);
    if (rc)
        return rc;
    std::string s;
    char line[512];
    for (auto& w : net.weights) {
        snprintf(line, sizeof(line), "weight %s dtype=%d scale=%.9g bytes=%zu dims=", w.name,
                 (int)w.dtype.type_enum, w.dtype.param.scale, w.size);
        s += line;
        for (int i = 0; i < w.layout.nr_dim; ++i)
            s += std::to_string(w.layout.dims[i]) + (i + 1 < w.layout.nr_dim ? "x" : "");
        s += "\n";
    }
    for (size_t mi = 0; mi < net.models.size(); ++mi) {
        DevModel& m = net.models[mi];
        snprintf(line, sizeof(line), "device_model %zu tensor_memory=%zu tensors=%zu instructions=%zu\n",
                 mi, m.tensor_memory, m.tensors.size(), m.instrs.size());
        s += line;
        for (auto& t : m.tensors) {
            snprintf(line, sizeof(line), "tensor %s offset=%zu bytes=%zu format=%d scale=%.9g dims=",
                     t.name, t.offset, t.size, (int)t.layout.format, t.dtype.param.scale);
            s += line;
            for (int i = 0; i < t.layout.nr_dim; ++i)
                s += std::to_string(t.layout.dims[i]) + (i + 1 < t.layout.nr_dim ? "x" : "");
            s += " stride=";
            for (int i = 0; i < t.layout.nr_dim; ++i)
                s += std::to_string(t.layout.stride[i]) + (i + 1 < t.layout.nr_dim ? "x" : "");
            s += "\n";
        }
        for (auto& ins : m.instrs) {
            if (!ins.is_opr)
                continue;
            s += "opr " + ins.op.symbol + " in=";
            for (auto* t : ins.op.inputs)
                s += std::string(t->name) + ",";
            s += " out=";
            for (auto* t : ins.op.outputs)
                s += std::string(t->name) + ",";
            s += " ws=" + std::to_string(ins.op.ws.offset) + "+" + std::to_string(ins.op.ws.size);
            s += "\n";
        }
        for (auto& io : m.inputs)
            s += std::string("input ") + io.tensor->name + "\n";
        for (auto& io : m.outputs)
            s += std::string("output ") + io.tensor->name + "\n";
    }
    if (s.size() + 1 > cap)
        return fail(TinyNN_ERROR_OUT_OF_RANGE, "summary needs %zu bytes", s.size() + 1);
    memcpy(out, s.c_str(), s.size() + 1);
    return TinyNN_SUCCESS;
}

int LITE_make_network(LiteNetwork* network, const LiteConfig config, const LiteNetworkIO io) {
    if (!network)
        return fail(TinyNN_ERROR_NULL_PTR, "network pointer is NULL");
    Network* net = new (std::nothrow) Network();
    if (!net)
        return fail(TinyNN_ERROR_MEMORY_MALLOC, "out of host memory");
    net->config = config;
    net->device_id = config.device_id >= 0 ? config.device_id : 0;
    for (size_t i = 0; i < io.input_size; ++i)
        if (io.inputs && io.inputs[i].name && !io.inputs[i].is_host)
            net->io_device_names.push_back(io.inputs[i].name);
    for (size_t i = 0; i < io.output_size; ++i)
        if (io.outputs && io.outputs[i].name && !io.outputs[i].is_host)
            net->io_device_names.push_back(io.outputs[i].name);
    net->use_graph = runtime_defaults().use_graph;
    net->profile = runtime_defaults().profile;
    *network = net;
    return TinyNN_SUCCESS;
}

int LITE_load_model_from_mem(LiteNetwork network, void* model_mem, size_t size) {
    if (!network || !model_mem)
        return fail(TinyNN_ERROR_NULL_PTR, "network or model pointer is NULL");
    Network* net = as_net(network);
    if (net->loaded)
        return fail(TinyNN_ERROR, "this network already holds a model");
    const int rc = parse_model(net, model_mem, size);
    return rc ? rc : upload_weights(net);
}

int LITE_load_model_with_shared_mem(LiteNetwork network, void* model_mem, size_t size) {
    // weights live in device memory either way, so sharing the host buffer changes nothing
    return LITE_load_model_from_mem(network, model_mem, size);
}

int LITE_load_model_from_path(LiteNetwork network, const char* model_path) {
    if (!network || !model_path)
        return fail(TinyNN_ERROR_NULL_PTR, "network or path is NULL");
    FILE* f = fopen(model_path, "rb");
    if (!f)
        return fail(TinyNN_ERROR_OPEN_FILE_ERROR, "cannot open %s", model_path);
    fseek(f, 0, SEEK_END);
    const long size = ftell(f);
    fseek(f, 0, SEEK_SET);
    Network* net = as_net(network);
    net->owned_model.resize(size > 0 ? (size_t)size : 0);
    const size_t got = size > 0 ? fread(net->owned_model.data(), 1, (size_t)size, f) : 0;
    fclose(f);
    if (size <= 0 || got != (size_t)size)
        return fail(TinyNN_ERROR_OPEN_FILE_ERROR, "short read of %s", model_path);
    return LITE_load_model_from_mem(network, net->owned_model.data(), net->owned_model.size());
}

int LITE_get_io_tensor(
        LiteNetwork network, const char* io_name, LiteTensorPhase phase, LiteTensor* tensor) {
    if (!network || !io_name || !tensor)
        return fail(TinyNN_ERROR_NULL_PTR, "input pointer is NULL");
    Network* net = as_net(network);
    if (!net->loaded)
        return fail(TinyNN_ERROR, "no model loaded");
    DevModel& m = net->models[net->active];
    for (int pass = 0; pass < 2; ++pass) {
        const bool input = pass == 0;
        if (input && phase == LITE_OUTPUT)
            continue;
        if (!input && phase == LITE_INPUT)
            continue;
        auto& v = input ? m.inputs : m.outputs;
        for (size_t i = 0; i < v.size(); ++i) {
            if (strcmp(v[i].tensor->name, io_name) == 0) {
                for (auto& h : net->handles)
                    if (h->is_input == input && h->index == (int)i) {
                        *tensor = h.get();
                        return TinyNN_SUCCESS;
                    }
                net->handles.emplace_back(new IoHandle{net, input, (int)i});
                *tensor = net->handles.back().get();
                return TinyNN_SUCCESS;
            }
        }
    }
    return fail(TinyNN_ERROR_NO_FOUND, "no input/output tensor named '%s'", io_name);
}

int LITE_get_tensor_total_size_in_byte(const LiteTensor tensor, size_t* size) {
    if (!tensor || !size)
        return fail(TinyNN_ERROR_NULL_PTR, "input pointer is NULL");
    IoSlot* s = slot_of(as_io(tensor));
    if (!s)
        return fail(TinyNN_ERROR_OUT_OF_RANGE, "stale tensor handle");
    *size = s->bytes;
    return TinyNN_SUCCESS;
}

int LITE_reset_tensor_memory(LiteTensor tensor, void* prepared_data, size_t data_length_in_byte) {
    if (!tensor || !prepared_data)
        return fail(TinyNN_ERROR_NULL_PTR, "input pointer is NULL");
    IoHandle* h = as_io(tensor);
    IoSlot* s = slot_of(h);
    if (!s)
        return fail(TinyNN_ERROR_OUT_OF_RANGE, "stale tensor handle");
    if (data_length_in_byte != s->bytes)
        return fail(TinyNN_ERROR, "reset tensor memory with not equal size %zu != %zu",
                    data_length_in_byte, s->bytes);
    if (!h->is_input)
        return fail(TinyNN_ERROR_NO_IMPLEMENT, "only input tensors take user memory");
    cudaPointerAttributes attr;
    bool is_dev = false;
    if (cudaPointerGetAttributes(&attr, prepared_data) == cudaSuccess)
        is_dev = attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
    else
        cudaGetLastError();
    if (is_dev && ((uintptr_t)prepared_data & 15))
        return fail(TinyNN_ERROR_INVALID_LAYOUT, "device input must be 16-byte aligned");
    s->user_ptr = prepared_data;
    s->user_is_device = is_dev;
    return TinyNN_SUCCESS;
}

int LITE_get_tensor_memory(const LiteTensor tensor, void** data) {
    if (!tensor || !data)
        return fail(TinyNN_ERROR_NULL_PTR, "input pointer is NULL");
    IoHandle* h = as_io(tensor);
    IoSlot* s = slot_of(h);
    if (!s)
        return fail(TinyNN_ERROR_OUT_OF_RANGE, "stale tensor handle");
    if (h->is_input) {
        if (!s->user_ptr)
            return fail(TinyNN_ERROR_NULL_PTR,
                        "the input tensor memory is NULL: call LITE_reset_tensor_memory first");
        *data = s->user_ptr;
        return TinyNN_SUCCESS;
    }
    int rc = init_model_memory(h->net);
    if (rc)
        return rc;
    if ((rc = wait(h->net)))  // results must be complete before the caller reads them
        return rc;
    *data = s->want_device ? s->tensor->ptr : s->host_stage;
    return TinyNN_SUCCESS;
}

static int lite_dtype(TinyNNDType t, LiteCDataType* out) {
    switch (t) {
        case TinyNN_FLOAT: *out = LITE_FLOAT; return 0;
        case TinyNN_FLOAT16: *out = LITE_HALF; return 0;
        case TinyNN_INT: *out = LITE_INT; return 0;
        case TinyNN_INT8: *out = LITE_INT8; return 0;
        case TinyNN_INT16: *out = LITE_INT16; return 0;
        case TinyNN_UINT8: *out = LITE_UINT8; return 0;
        default:
            // quantised dtypes have no lite counterpart (runtime/src/lite/tensor.c:11-40)
            return TinyNN_ERROR_OUT_OF_RANGE;
    }
}

int LITE_get_tensor_layout(const LiteTensor tensor, LiteLayout* layout) {
    if (!tensor || !layout)
        return fail(TinyNN_ERROR_NULL_PTR, "input pointer is NULL");
    IoSlot* s = slot_of(as_io(tensor));
    if (!s)
        return fail(TinyNN_ERROR_OUT_OF_RANGE, "stale tensor handle");
    const int rc = lite_dtype(s->tensor->dtype.type_enum, &layout->data_type);
    if (rc)
        return fail(rc, "failed convert tinynn dtype to lite");
    layout->ndim = s->tensor->layout.nr_dim;
    for (size_t i = 0; i < layout->ndim; ++i)
        layout->shapes[i] = s->tensor->layout.dims[i];
    return TinyNN_SUCCESS;
}

int LITE_set_tensor_layout(LiteTensor tensor, const LiteLayout layout) {
    if (!tensor)
        return fail(TinyNN_ERROR_NULL_PTR, "input pointer is NULL");
    IoHandle* h = as_io(tensor);
    Network* net = h->net;
    // pick the DeviceModel (shape variant) whose tensor matches (tensor.c:78-91)
    for (size_t mi = 0; mi < net->models.size(); ++mi) {
        auto& v = h->is_input ? net->models[mi].inputs : net->models[mi].outputs;
        if ((size_t)h->index >= v.size())
            continue;
        const Tensor* t = v[h->index].tensor;
        bool same = (size_t)t->layout.nr_dim == layout.ndim;
        for (size_t i = 0; same && i < layout.ndim; ++i)
            same = t->layout.dims[i] == layout.shapes[i];
        if (same) {
            if (wait(net))
                return TinyNN_ERROR_RUNTIME;
            net->active = (int)mi;
            return TinyNN_SUCCESS;
        }
    }
    return fail(TinyNN_ERROR_INVALID_LAYOUT, "no device model has this layout");
}

int LITE_destroy_tensor(LiteTensor) {
    return TinyNN_SUCCESS;
}

int LITE_forward(const LiteNetwork network) {
    if (!network)
        return fail(TinyNN_ERROR_NULL_PTR, "network is NULL");
    return forward(as_net(network));
}

int LITE_wait(const LiteNetwork network) {
    if (!network)
        return fail(TinyNN_ERROR_NULL_PTR, "network is NULL");
    return wait(as_net(network));
}

static int io_name(const LiteNetwork network, size_t index, const char** name, bool input) {
    if (!network || !name)
        return fail(TinyNN_ERROR_NULL_PTR, "input pointer is NULL");
    Network* net = as_net(network);
    if (!net->loaded)
        return fail(TinyNN_ERROR, "no model loaded");
    auto& v = input ? net->models[net->active].inputs : net->models[net->active].outputs;
    if (index >= v.size())
        return fail(TinyNN_ERROR_OUT_OF_RANGE, "index %zu out of range", index);
    *name = v[index].tensor->name;
    return TinyNN_SUCCESS;
}
int LITE_get_input_name(const LiteNetwork network, size_t index, const char** name) {
    return io_name(network, index, name, true);
}
int LITE_get_output_name(const LiteNetwork network, size_t index, const char** name) {
    return io_name(network, index, name, false);
}

static int all_names(const LiteNetwork network, size_t* size, const char** name, bool input) {
    if (!network)
        return fail(TinyNN_ERROR_NULL_PTR, "input pointer is NULL");
    Network* net = as_net(network);
    if (!net->loaded)
        return fail(TinyNN_ERROR, "no model loaded");
    auto& v = input ? net->models[net->active].inputs : net->models[net->active].outputs;
    if (size)
        *size = v.size();
    if (name)
        for (size_t i = 0; i < v.size(); ++i)
            name[i] = v[i].tensor->name;
    return TinyNN_SUCCESS;
}
int LITE_get_all_input_name(const LiteNetwork network, size_t* size, const char** name) {
    return all_names(network, size, name, true);
}
int LITE_get_all_output_name(const LiteNetwork network, size_t* size, const char** name) {
    return all_names(network, size, name, false);
}

int LITE_share_runtime_memroy(LiteNetwork src_network, LiteNetwork dst_network) {
    if (!src_network || !dst_network)
        return fail(TinyNN_ERROR_NULL_PTR, "network is NULL");
    Network* src = as_net(src_network);
    Network* dst = as_net(dst_network);
    if (src->arena->ptr || dst->arena->ptr)
        return fail(TinyNN_ERROR, "shared runtime memory should be called before model run");
    if (src->device_id != dst->device_id)
        return fail(TinyNN_ERROR, "networks live on different devices");
    // one arena sized for the larger of the two; both networks must then run on one
    // stream's worth of ordering, which the caller gets by waiting between forwards
    src->arena->bytes = src->arena_need > dst->arena_need ? src->arena_need : dst->arena_need;
    dst->arena = src->arena;
    return TinyNN_SUCCESS;
}

int LITE_destroy_network(LiteNetwork network) {
    if (!network)
        return TinyNN_ERROR_NULL_PTR;
    Network* net = as_net(network);
    cudaSetDevice(net->device_id);
    if (net->stream)
        cudaStreamSynchronize(net->stream);
    for (auto& m : net->models) {
        if (net->profile)
            for (auto& ins : m.instrs)
                if (ins.is_opr && ins.op.ms_count)
                    log_at(LITE_WARN, "profile %-90s %8.4f ms\n", ins.op.symbol.c_str(),
                           ins.op.ms_total / ins.op.ms_count);
        for (auto& g : m.graphs)
            cudaGraphExecDestroy(g.exec);
        m.graphs.clear();
        for (auto& o : m.outputs)
            if (o.host_stage)
                cudaFreeHost(o.host_stage);
    }
    if (net->weight_arena)
        cudaFree(net->weight_arena);
    for (int i = 0; i < Network::kCopyStreams; ++i) {
        if (net->copy_stream[i])
            cudaStreamDestroy(net->copy_stream[i]);
        if (net->copy_join[i])
            cudaEventDestroy(net->copy_join[i]);
    }
    if (net->copy_fork)
        cudaEventDestroy(net->copy_fork);
    if (net->stream)
        cudaStreamDestroy(net->stream);
    delete net;
    return TinyNN_SUCCESS;
}

// ---- additions without a counterpart in the reference ----
int mb200_lite_stream(const LiteNetwork network, void** stream) {
    if (!network || !stream)
        return fail(TinyNN_ERROR_NULL_PTR, "input pointer is NULL");
    *stream = as_net(network)->stream;
    return TinyNN_SUCCESS;
}

int mb200_lite_set_kernel_tables(
        LiteNetwork network, const void* kernel_table, int nr_kernels, const void* init_table,
        int nr_init) {
    const KernelFunc* kernels = (const KernelFunc*)kernel_table;
    const InitFunc* init_kernels = (const InitFunc*)init_table;
    if (!network || (nr_kernels > 0 && !kernels) || (nr_init > 0 && !init_kernels))
        return fail(TinyNN_ERROR_NULL_PTR, "input pointer is NULL");
    Network* net = as_net(network);
    if (net->loaded)
        return fail(TinyNN_ERROR, "kernel tables must be registered before the model is loaded");
    net->ext_kernels.assign(kernels, kernels + (nr_kernels > 0 ? nr_kernels : 0));
    net->ext_inits.assign(init_kernels, init_kernels + (nr_init > 0 ? nr_init : 0));
    return TinyNN_SUCCESS;
}

int mb200_lite_set_option(LiteNetwork network, const char* name, int value) {
    if (!network || !name)
        return fail(TinyNN_ERROR_NULL_PTR, "input pointer is NULL");
    Network* net = as_net(network);
    if (strcmp(name, "use_graph") == 0) {
        if (wait(net))
            return TinyNN_ERROR_RUNTIME;
        net->use_graph = value != 0;
        return TinyNN_SUCCESS;
    }
    if (strcmp(name, "profile") == 0) {
        net->profile = value != 0;
        return TinyNN_SUCCESS;
    }
    return fail(TinyNN_ERROR_OUT_OF_RANGE, "unknown option '%s'", name);
}

int mb200_lite_set_profile(LiteNetwork network, int enable) {
    if (!network)
        return fail(TinyNN_ERROR_NULL_PTR, "network is NULL");
    as_net(network)->profile = enable != 0;
    return TinyNN_SUCCESS;
}

int mb200_lite_profile(const LiteNetwork network, char* out, size_t cap) {
    if (!network || !out || !cap)
        return fail(TinyNN_ERROR_NULL_PTR, "input pointer is NULL");
    Network* net = as_net(network);
    if (!net->loaded)
        return fail(TinyNN_ERROR, "no model loaded");
    std::string s;
    char line[512];
    for (auto& ins : net->models[net->active].instrs) {
        if (!ins.is_opr)
            continue;
        snprintf(line, sizeof(line), "%s %s %.6f %d\n", ins.op.name.c_str(), ins.op.symbol.c_str(),
                 ins.op.ms_count ? ins.op.ms_total / ins.op.ms_count : 0.f, ins.op.ms_count);
        s += line;
    }
    if (s.size() + 1 > cap)
        return fail(TinyNN_ERROR_OUT_OF_RANGE, "profile needs %zu bytes", s.size() + 1);
    memcpy(out, s.c_str(), s.size() + 1);
    return TinyNN_SUCCESS;
}

int LITE_get_device_id(const LiteNetwork network, int* device_id) {
    if (!network || !device_id)
        return fail(TinyNN_ERROR_NULL_PTR, "input pointer is NULL");
    *device_id = as_net(network)->device_id;
    return TinyNN_SUCCESS;
}

int LITE_set_device_id(LiteNetwork network, int device_id) {
    if (!network)
        return fail(TinyNN_ERROR_NULL_PTR, "network is NULL");
    Network* net = as_net(network);
    if (net->loaded)
        return fail(TinyNN_ERROR, "the device must be chosen before the model is loaded");
    if (device_id < 0)
        return fail(TinyNN_ERROR_OUT_OF_RANGE, "device id %d", device_id);
    net->device_id = device_id;
    return TinyNN_SUCCESS;
}

int LITE_get_device_type(const LiteNetwork network, LiteDeviceType* device_type) {
    if (!network || !device_type)
        return fail(TinyNN_ERROR_NULL_PTR, "input pointer is NULL");
    *device_type = LITE_CUDA;
    return TinyNN_SUCCESS;
}

int LITE_get_tensor_device_type(const LiteTensor tensor, LiteDeviceType* device_type) {
    if (!tensor || !device_type)
        return fail(TinyNN_ERROR_NULL_PTR, "input pointer is NULL");
    IoHandle* h = as_io(tensor);
    IoSlot* s = slot_of(h);
    if (!s)
        return fail(TinyNN_ERROR_OUT_OF_RANGE, "stale tensor handle");
    const bool dev = h->is_input ? s->user_is_device : s->want_device;
    *device_type = dev ? LITE_CUDA : LITE_CPU;
    return TinyNN_SUCCESS;
}

}  // extern "C"
