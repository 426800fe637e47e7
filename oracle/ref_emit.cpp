// TEST INFRASTRUCTURE (checker only; never linked into or called by the product).
//
// Drives the UNMODIFIED MegCC KernelGen registry (compiled from the reference
// sources where they lie, see oracle/Makefile) and writes the C source of the
// kernel the reference itself would pick on x86 (Arch::BAREMETAL: the
// GeneralIntrinsic list followed by the BareMetal list, first IsAvailable wins;
// compiler/lib/KernelGen/KernelGen.cpp:100-125).
//
// Input: a spec file, one kernel per line (see oracle/ref_specs.txt).
// Output: <outdir>/<symbol>.c for every spec and <outdir>/symbols.txt listing
//         "<spec line> => <symbol>".
//
// The attribute names follow the reference's own unit-test harness
// (compiler/test/kernel/common/src/cc_fill_attr.cpp:253-292,
//  compiler/test/kernel/common/src/cc_proxy_utils.h:37-106).
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <set>
#include <sstream>
#include <string>
#include <unordered_map>
#include <vector>

#include "compiler/Common/TContext.h"
#include "compiler/KernelGen/KernelGen.h"

using namespace megcc;
using KernType = KernelGen::KernelPack::KernType;

static uint32_t f2u(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
}

static CCOperand make_operand(
        const std::string& base, std::vector<size_t> shape, float scale = 1.f) {
    CCOperand op;
    op.shape = shape;
    if (base == "qsi8" || base == "qsi32") {
        std::stringstream ss;
        ss << base << "<" << f2u(scale) << ":" << scale << ">";
        op.dtype = ss.str();
        op.scale = scale;
    } else {
        op.dtype = base;
    }
    return op;
}

struct Emitted {
    std::string symbol, body;
    // internal kernels the chosen kernel depends on (symbol -> C text), emitted once each as
    // files of their own, as the reference's exporter does
    std::vector<std::pair<std::string, std::string>> deps;
};

static void collect_deps(
        const std::vector<KernelGen::KernelObj>& objs,
        std::vector<std::pair<std::string, std::string>>& out) {
    for (auto& d : objs) {
        collect_deps(d.kernel_dep, out);
        std::stringstream ss;
        ss << KernelGen::GenCommonInclude() << "\n" << d.kernel_body << "\n";
        out.push_back({d.kernel_symbol, ss.str()});
    }
}

static bool pick(
        KernType type, std::unordered_map<std::string, CCAttr>& attrs, Emitted& out) {
    CodeGenContext ctx(attrs);
    auto kerns = KernelGen::KernelPack::GetKernel(type, KernelGen::Arch::BAREMETAL).first;
    for (auto* k : kerns) {
        if (k->IsAvailable(&ctx)) {
            out.symbol = k->GetKernelSymbol(&ctx);
            collect_deps(k->GetDependInternalSymbol(&ctx), out.deps);
            std::stringstream ss;
            ss << KernelGen::GenCommonInclude() << "\n";
            ss << k->GetKernelBody(&ctx) << "\n";
            // the weight-preprocessing and workspace functions of the same kernel (the fp32
            // GEMM-based kernels need both; for the others these are the trivial defaults)
            ss << k->GetInitBody(&ctx) << "\n";
            ss << k->GetWorkspaceBody(&ctx) << "\n";
            out.body = ss.str();
            return true;
        }
    }
    return false;
}

int main(int argc, char** argv) {
    if (argc != 3) {
        fprintf(stderr, "usage: %s <specs.txt> <outdir>\n", argv[0]);
        return 2;
    }
    std::ifstream in(argv[1]);
    std::string outdir = argv[2];
    std::ofstream symfile(outdir + "/symbols.txt");
    std::set<std::string> done;
    std::string line;
    int nline = 0;
    while (std::getline(in, line)) {
        ++nline;
        if (line.empty() || line[0] == '#')
            continue;
        std::stringstream ls(line);
        std::string kind;
        ls >> kind;
        std::unordered_map<std::string, CCAttr> attrs;
        Emitted em;
        bool ok = false;
        if (kind == "conv") {
            // conv <kh> <kw> <sh> <sw> <ph> <pw> <sparse> <nonline> <bias 0|1>
            uint32_t kh, kw, sh, sw, ph, pw;
            std::string sparse, nonline;
            int bias;
            ls >> kh >> kw >> sh >> sw >> ph >> pw >> sparse >> nonline >> bias;
            attrs["kernel_h"] = CCAttr(kh);
            attrs["kernel_w"] = CCAttr(kw);
            attrs["stride_h"] = CCAttr(sh);
            attrs["stride_w"] = CCAttr(sw);
            attrs["pad_h"] = CCAttr(ph);
            attrs["pad_w"] = CCAttr(pw);
            attrs["dilate_h"] = CCAttr((uint32_t)1);
            attrs["dilate_w"] = CCAttr((uint32_t)1);
            attrs["sparse"] = CCAttr(sparse);
            attrs["format"] = CCAttr("NCHW");
            attrs["mode"] = CCAttr("CROSS_CORRELATION");
            attrs["nonlineMode"] = CCAttr(nonline);
            attrs["compute_mode"] = CCAttr("DEFAULT");
            // shapes only steer IsAvailable / the symbol; the emitted kernel reads
            // all extents from the Tensor layouts at run time.
            size_t c = 8;
            attrs["operand:0"] = CCAttr(make_operand("qsi8", {1, c, 16, 16}));
            if (sparse == "DENSE")
                attrs["operand:1"] = CCAttr(make_operand("qsi8", {c, c, kh, kw}));
            else
                attrs["operand:1"] = CCAttr(make_operand("qsi8", {c, 1, 1, kh, kw}));
            if (bias) {
                attrs["operand:2"] = CCAttr(make_operand("qsi32", {1, c, 1, 1}));
            } else {
                attrs["operand:2"] = CCAttr(make_operand("qsi32", {}));
            }
            // no z operand: MGBToKernel never fills it
            // (compiler/lib/Conversion/MGBToKernel/MGBToKernel.cpp:245-256)
            attrs["operand:3"] = CCAttr(make_operand("qsi8", {1, c, 16, 16}));
            attrs["nr_operands"] = CCAttr((int)4);
            ok = pick(KernType::ConvKernel, attrs, em);
        } else if (kind == "conv44") {
            // conv44 <kh> <kw> <sh> <sw> <ph> <pw> <DENSE|GROUP|HYBRID> <nonline> <bias 0|1>
            // format NCHW44: tensors [N][C/4][H][W][4]; GROUP is channel-wise; HYBRID is the
            // first layer with an NCHW input, which the reference names NCHW_NCHW44
            // (compiler/lib/KernelGen/BareMetal/ConvKernel.cpp:111-121)
            uint32_t kh, kw, sh, sw, ph, pw;
            std::string sparse, nonline;
            int bias;
            ls >> kh >> kw >> sh >> sw >> ph >> pw >> sparse >> nonline >> bias;
            const bool hybrid = sparse == "HYBRID";
            attrs["kernel_h"] = CCAttr(kh);
            attrs["kernel_w"] = CCAttr(kw);
            attrs["stride_h"] = CCAttr(sh);
            attrs["stride_w"] = CCAttr(sw);
            attrs["pad_h"] = CCAttr(ph);
            attrs["pad_w"] = CCAttr(pw);
            attrs["dilate_h"] = CCAttr((uint32_t)1);
            attrs["dilate_w"] = CCAttr((uint32_t)1);
            attrs["sparse"] = CCAttr(hybrid ? std::string("DENSE") : sparse);
            attrs["format"] = CCAttr("NCHW44");
            attrs["mode"] = CCAttr("CROSS_CORRELATION");
            attrs["nonlineMode"] = CCAttr(nonline);
            attrs["compute_mode"] = CCAttr("DEFAULT");
            if (hybrid) {
                attrs["operand:0"] = CCAttr(make_operand("qsi8", {1, 3, 16, 16}));
                attrs["operand:1"] = CCAttr(make_operand("qsi8", {2, kh, kw, 3, 4}));
            } else if (sparse == "DENSE") {
                attrs["operand:0"] = CCAttr(make_operand("qsi8", {1, 2, 16, 16, 4}));
                attrs["operand:1"] = CCAttr(make_operand("qsi8", {2, 2, kh, kw, 4, 4}));
            } else {
                attrs["operand:0"] = CCAttr(make_operand("qsi8", {1, 2, 16, 16, 4}));
                attrs["operand:1"] = CCAttr(make_operand("qsi8", {2, 1, 1, kh, kw, 4}));
            }
            attrs["operand:2"] = bias ? CCAttr(make_operand("qsi32", {1, 2, 1, 1, 4}))
                                      : CCAttr(make_operand("qsi32", {}));
            attrs["operand:3"] = CCAttr(make_operand("qsi8", {1, 2, 16, 16, 4}));
            attrs["nr_operands"] = CCAttr((int)4);
            ok = pick(KernType::ConvKernel, attrs, em);
        } else if (kind == "pool") {
            // pool <mode> <wh> <ww> <sh> <sw> <ph> <pw>
            std::string mode;
            uint32_t wh, ww, sh, sw, ph, pw;
            ls >> mode >> wh >> ww >> sh >> sw >> ph >> pw;
            attrs["mode"] = CCAttr(mode);
            attrs["format"] = CCAttr("NCHW");
            attrs["window_h"] = CCAttr(wh);
            attrs["window_w"] = CCAttr(ww);
            attrs["stride_h"] = CCAttr(sh);
            attrs["stride_w"] = CCAttr(sw);
            attrs["pad_h"] = CCAttr(ph);
            attrs["pad_w"] = CCAttr(pw);
            attrs["operand:0"] = CCAttr(make_operand("qsi8", {1, 8, 16, 16}));
            attrs["operand:1"] = CCAttr(make_operand("qsi8", {1, 8, 8, 8}));
            attrs["nr_operands"] = CCAttr((int)2);
            ok = pick(KernType::PoolingKernel, attrs, em);
        } else if (kind == "qelem") {
            // qelem <QADD|QFUSE_ADD_RELU|QMUL|QRELU>
            std::string mode;
            ls >> mode;
            attrs["mode"] = CCAttr(mode);
            int n = (mode == "QRELU") ? 2 : 3;
            for (int i = 0; i < n; ++i)
                attrs["operand:" + std::to_string(i)] =
                        CCAttr(make_operand("qsi8", {1, 8, 16, 16}));
            attrs["nr_operands"] = CCAttr(n);
            ok = pick(KernType::ElemwiseMultiKernel, attrs, em);
        } else if (kind == "typecvt") {
            // typecvt <src dtype> <dst dtype>
            std::string s, d;
            ls >> s >> d;
            attrs["operand:0"] = CCAttr(make_operand(s, {1, 8, 16, 16}));
            attrs["operand:1"] = CCAttr(make_operand(d, {1, 8, 16, 16}));
            attrs["nr_operands"] = CCAttr((int)2);
            ok = pick(KernType::TypeCvtKernel, attrs, em);
        } else if (kind == "convf32") {
            // convf32 <kh> <kw> <sh> <sw> <ph> <pw> <nonline> <bias 0|1> <ic> <oc> <hw>
            uint32_t kh, kw, sh, sw, ph, pw;
            std::string nonline;
            int bias;
            size_t ic, oc, hw;
            ls >> kh >> kw >> sh >> sw >> ph >> pw >> nonline >> bias >> ic >> oc >> hw;
            attrs["kernel_h"] = CCAttr(kh);
            attrs["kernel_w"] = CCAttr(kw);
            attrs["stride_h"] = CCAttr(sh);
            attrs["stride_w"] = CCAttr(sw);
            attrs["pad_h"] = CCAttr(ph);
            attrs["pad_w"] = CCAttr(pw);
            attrs["dilate_h"] = CCAttr((uint32_t)1);
            attrs["dilate_w"] = CCAttr((uint32_t)1);
            attrs["sparse"] = CCAttr("DENSE");
            attrs["format"] = CCAttr("NCHW");
            attrs["mode"] = CCAttr("CROSS_CORRELATION");
            attrs["nonlineMode"] = CCAttr(nonline);
            attrs["compute_mode"] = CCAttr("DEFAULT");
            const size_t oh = (hw + 2 * ph - kh) / sh + 1;
            attrs["operand:0"] = CCAttr(make_operand("f32", {1, ic, hw, hw}));
            attrs["operand:1"] = CCAttr(make_operand("f32", {oc, ic, kh, kw}));
            attrs["operand:2"] = bias ? CCAttr(make_operand("f32", {1, oc, 1, 1}))
                                      : CCAttr(make_operand("f32", {}));
            attrs["operand:3"] = CCAttr(make_operand("f32", {1, oc, oh, oh}));
            attrs["nr_operands"] = CCAttr((int)4);
            ok = pick(KernType::ConvKernel, attrs, em);
        } else if (kind == "matmulf32") {
            // matmulf32 <m> <n> <k>
            size_t m, n, k;
            ls >> m >> n >> k;
            attrs["transposeA"] = CCAttr(false);
            attrs["transposeB"] = CCAttr(false);
            attrs["format"] = CCAttr("DEFAULT");
            attrs["compute_mode"] = CCAttr("DEFAULT");
            attrs["operand:0"] = CCAttr(make_operand("f32", {m, k}));
            attrs["operand:1"] = CCAttr(make_operand("f32", {k, n}));
            attrs["operand:2"] = CCAttr(make_operand("f32", {m, n}));
            attrs["nr_operands"] = CCAttr((int)3);
            ok = pick(KernType::MatrixMulKernel, attrs, em);
        } else if (kind == "elemf32") {
            // elemf32 <MODE> <nr inputs>
            std::string mode;
            int n;
            ls >> mode >> n;
            attrs["mode"] = CCAttr(mode);
            for (int i = 0; i <= n; ++i)
                attrs["operand:" + std::to_string(i)] =
                        CCAttr(make_operand("f32", {1, 8, 16, 16}));
            attrs["nr_operands"] = CCAttr(n + 1);
            ok = pick(KernType::ElemwiseKernel, attrs, em);
        } else if (kind == "concatf32") {
            // concatf32 <axis> <nr inputs>
            int axis, n;
            ls >> axis >> n;
            attrs["axis"] = CCAttr(axis);
            for (int i = 0; i < n; ++i)
                attrs["operand:" + std::to_string(i)] =
                        CCAttr(make_operand("f32", {1, 8, 16, 16}));
            attrs["operand:" + std::to_string(n)] =
                    CCAttr(make_operand("f32", {1, (size_t)(8 * n), 16, 16}));
            attrs["nr_operands"] = CCAttr(n + 1);
            ok = pick(KernType::ConcatKernel, attrs, em);
        } else if (kind == "resizef32") {
            // resizef32 <imode>
            std::string imode;
            ls >> imode;
            attrs["imode"] = CCAttr(imode);
            attrs["format"] = CCAttr("NCHW");
            attrs["operand:0"] = CCAttr(make_operand("f32", {1, 8, 16, 16}));
            attrs["operand:1"] = CCAttr(make_operand("f32", {1, 8, 32, 32}));
            attrs["nr_operands"] = CCAttr((int)2);
            ok = pick(KernType::ResizeKernel, attrs, em);
        } else if (kind == "poolf32") {
            // poolf32 <mode> <wh> <ww> <sh> <sw> <ph> <pw>
            std::string mode;
            uint32_t wh, ww, sh, sw, ph, pw;
            ls >> mode >> wh >> ww >> sh >> sw >> ph >> pw;
            attrs["mode"] = CCAttr(mode);
            attrs["format"] = CCAttr("NCHW");
            attrs["window_h"] = CCAttr(wh);
            attrs["window_w"] = CCAttr(ww);
            attrs["stride_h"] = CCAttr(sh);
            attrs["stride_w"] = CCAttr(sw);
            attrs["pad_h"] = CCAttr(ph);
            attrs["pad_w"] = CCAttr(pw);
            attrs["operand:0"] = CCAttr(make_operand("f32", {1, 8, 16, 16}));
            attrs["operand:1"] = CCAttr(make_operand("f32", {1, 8, 16, 16}));
            attrs["nr_operands"] = CCAttr((int)2);
            ok = pick(KernType::PoolingKernel, attrs, em);
        } else {
            fprintf(stderr, "line %d: unknown kind '%s'\n", nline, kind.c_str());
            return 1;
        }
        if (!ok) {
            fprintf(stderr, "line %d: no reference kernel available: %s\n", nline,
                    line.c_str());
            return 1;
        }
        symfile << line << " => " << em.symbol << "\n";
        if (done.insert(em.symbol).second) {
            std::ofstream f(outdir + "/" + em.symbol + ".c");
            f << em.body;
        }
        for (auto& d : em.deps)
            if (done.insert(d.first).second) {
                std::ofstream f(outdir + "/" + d.first + ".c");
                f << d.second;
            }
    }
    return 0;
}
