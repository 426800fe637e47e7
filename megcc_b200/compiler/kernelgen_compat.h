// The KernelGen plugin interface that the CUDA kernel pack implements.
//
// Inside a MegCC checkout, build with -DMEGCC_B200_IN_MEGCC_TREE and the reference's own
// headers are used (compiler/include/compiler/KernelGen/KernelGen.h:75-136 for KernelFunc,
// compiler/include/compiler/Common/TContext.h:11-243 for TContext / CCOperand / CCAttr),
// so the classes in cuda_kernel_pack.h derive from the very same base the registry walks.
// Stand-alone, the declarations below provide the same names, members and virtual-function
// order, trimmed to what a kernel pack touches.
#pragma once

#ifdef MEGCC_B200_IN_MEGCC_TREE
#include "compiler/KernelGen/KernelGen.h"
#else

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <sstream>
#include <string>
#include <vector>

namespace megcc {

// one operand of an operator: static shape, dtype string ("qsi8<bits:scale>", "qsi32<..>",
// "f32", ...) and quantisation scale (-1 when not quantised)
struct CCOperand {
    std::vector<size_t> shape;
    std::string dtype;
    float scale = -1.f;
};

// attribute bag handed to every KernelFunc
struct TContext {
    virtual int8_t getAttrInt8(const std::string& attrName) = 0;
    virtual uint8_t getAttrUInt8(const std::string& attrName) = 0;
    virtual int32_t getAttrInt(const std::string& attrName) = 0;
    virtual uint32_t getAttrUInt(const std::string& attrName) = 0;
    virtual uint64_t getAttrUInt64(const std::string& attrName) = 0;
    virtual int64_t getAttrInt64(const std::string& attrName) = 0;
    virtual float getAttrFloat(const std::string& attrName) = 0;
    virtual double getAttrDouble(const std::string& attrName) = 0;
    virtual std::string getAttrStr(const std::string& attrName) = 0;
    virtual CCOperand getAttrOprand(const std::string& attrName) = 0;
    virtual bool getAttrBool(const std::string& attrName) = 0;
    virtual bool haveAttr(const std::string& attrName) = 0;
    virtual ~TContext() = default;
};

// a concrete attribute bag for the stand-alone build: integers, floats, strings, operands
class CodeGenContext final : public TContext {
public:
    void setInt(const std::string& k, int64_t v) { ints_[k] = v; }
    void setFloat(const std::string& k, double v) { floats_[k] = v; }
    void setStr(const std::string& k, const std::string& v) { strs_[k] = v; }
    void setOperand(const std::string& k, const CCOperand& v) { operands_[k] = v; }

    int8_t getAttrInt8(const std::string& k) override { return (int8_t)geti(k); }
    uint8_t getAttrUInt8(const std::string& k) override { return (uint8_t)geti(k); }
    int32_t getAttrInt(const std::string& k) override { return (int32_t)geti(k); }
    uint32_t getAttrUInt(const std::string& k) override { return (uint32_t)geti(k); }
    uint64_t getAttrUInt64(const std::string& k) override { return (uint64_t)geti(k); }
    int64_t getAttrInt64(const std::string& k) override { return geti(k); }
    float getAttrFloat(const std::string& k) override { return (float)getf(k); }
    double getAttrDouble(const std::string& k) override { return getf(k); }
    std::string getAttrStr(const std::string& k) override {
        auto it = strs_.find(k);
        if (it == strs_.end())
            missing(k);
        return it->second;
    }
    CCOperand getAttrOprand(const std::string& k) override {
        auto it = operands_.find(k);
        if (it == operands_.end())
            missing(k);
        return it->second;
    }
    bool getAttrBool(const std::string& k) override { return geti(k) != 0; }
    bool haveAttr(const std::string& k) override {
        return ints_.count(k) || floats_.count(k) || strs_.count(k) || operands_.count(k);
    }

private:
    std::map<std::string, int64_t> ints_;
    std::map<std::string, double> floats_;
    std::map<std::string, std::string> strs_;
    std::map<std::string, CCOperand> operands_;
    [[noreturn]] static void missing(const std::string& k) {
        // the reference aborts on a missing attribute as well (TContext.h:226-233)
        fprintf(stderr, "not find CCAttr %s\n", k.c_str());
        abort();
    }
    int64_t geti(const std::string& k) {
        auto it = ints_.find(k);
        if (it == ints_.end())
            missing(k);
        return it->second;
    }
    double getf(const std::string& k) {
        auto it = floats_.find(k);
        if (it == floats_.end())
            missing(k);
        return it->second;
    }
};

namespace KernelGen {

enum KernelPriority { LOW = 0, NORMAL = 1, HIGH = 2 };

// the five fixed pieces of C text every generated function is assembled from
// (compiler/lib/KernelGen/KernelGen.cpp:130-153)
inline std::string GenCommonRet() {
    return "TinyNNStatus";
}
inline std::string GenCommonCall() {
    return "(Tensor** inputs, int nr_input, Tensor** outputs, int nr_output, "
           "const Workspace* workspace, const RuntimeOpt* opt)";
}
inline std::string GenCommonInitCall() {
    return "(Tensor** inputs, int nr_input, Tensor* out_weights, int* nr_out_weight, "
           "const RuntimeOpt* opt)";
}
inline std::string GenCommonWorkspaceCall() {
    return "(Tensor** inputs, int nr_input, int nr_thread, size_t* workspace)";
}

struct KernelObj {
    std::string kernel_symbol, kernel_body, guard_begin, guard_end;
    std::vector<KernelObj> kernel_dep;
    std::vector<uint8_t> kernel_bin;
};

struct KernelFunc {
    virtual bool IsAvailable(TContext* context) const = 0;
    virtual KernelPriority GetPriority() const { return KernelPriority::NORMAL; }
    virtual std::string GetKernelSymbol(TContext* context) const = 0;
    virtual std::string GetKernelSignature(TContext* context) const {
        return GetKernelSymbol(context) + GenCommonCall();
    }
    virtual std::string GetKernelBody(TContext* context) const = 0;
    virtual bool IsCVAvailable(TContext*) const { return false; }
    virtual std::string GetCVKernelSymbol(TContext*) const { return ""; }
    virtual std::string GetCVKernelSignature(TContext*) const { return ""; }
    virtual std::string GetCVKernelBody(TContext*) const { return ""; }
    virtual std::string GetInitSymbol(TContext* context) const {
        return GetKernelSymbol(context) + "_init";
    }
    virtual std::string GetInitSignature(TContext* context) const {
        return GetInitSymbol(context) + GenCommonInitCall();
    }
    virtual std::string GetInitBody(TContext* context) const {
        return GenCommonRet() + " " + GetInitSignature(context) +
               "{ if (nr_out_weight) { *nr_out_weight = 0; } return TinyNN_SUCCESS; }";
    }
    virtual std::string GetWorkspaceSymbol(TContext* context) const {
        return GetKernelSymbol(context) + "_workspace";
    }
    virtual std::string GetWorkspaceSignature(TContext* context) const {
        return GetWorkspaceSymbol(context) + GenCommonWorkspaceCall();
    }
    virtual std::string GetWorkspaceBody(TContext* context) const {
        return GenCommonRet() + " " + GetWorkspaceSignature(context) +
               "{ return TinyNN_SUCCESS; }";
    }
    virtual std::string GetWorkspaceBodyAndJitExec(TContext* context) const {
        return GetWorkspaceBody(context);
    }
    virtual std::string GetBodyGuardBegin(TContext*) const { return ""; }
    virtual std::string GetBodyGuardEnd(TContext*) const { return ""; }
    virtual std::vector<KernelObj> GetDependInternalSymbol(TContext*) const { return {}; }
};

struct KernelPack {
    // the kernel families the CUDA pack answers for; numbering follows
    // compiler/include/compiler/KernelGen/KernelGen.h:160-193
    enum class KernType {
        Unknow = 0,
        ConvKernel = 1,
        ElemwiseKernel = 2,
        ElemwiseMultiKernel = 3,
        PoolingKernel = 4,
        MatrixMulKernel = 5,
        RelayoutKernel = 7,
        TypeCvtKernel = 13,
        ResizeKernel = 19,
        ConcatKernel = 25,
    };
};

}  // namespace KernelGen
}  // namespace megcc
#endif  // MEGCC_B200_IN_MEGCC_TREE
