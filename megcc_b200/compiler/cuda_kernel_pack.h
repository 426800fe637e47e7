// The CUDA (sm_100a) architecture of KernelGen: KernelFunc implementations whose generated
// "kernel body" is a small host C stub with the reference's uniform kernel signature that
// launches the pre-built sm_100a kernel through the C ABI of libmegcc_b200.so.
//
// Mirrors the per-arch packs of the reference (compiler/lib/KernelGen/BareMetal/KernelPack.cpp
// :38-116): static singletons, order in the returned vector = priority, first IsAvailable wins.
#pragma once
#include <string>
#include <vector>

#include "kernelgen_compat.h"

namespace megcc {
namespace KernelGen {
namespace Cuda {

// qint8 ConvBias, activations NHWC. Admits a subset of what BareMetal::ConvGeneral admits
// (compiler/lib/KernelGen/BareMetal/ConvKernel.cpp:16-46).
class ConvBiasQS8 : public KernelFunc {
public:
    bool IsAvailable(TContext* ctx) const override;
    std::string GetKernelSymbol(TContext* ctx) const override;
    std::string GetKernelBody(TContext* ctx) const override;
    std::string GetInitBody(TContext* ctx) const override;
    std::string GetWorkspaceBody(TContext* ctx) const override;
    // bytes of device scratch the kernel needs for the operator `ctx` describes
    size_t WorkspaceBytes(TContext* ctx) const;
};

class PoolingQS8 : public KernelFunc {
public:
    bool IsAvailable(TContext* ctx) const override;
    std::string GetKernelSymbol(TContext* ctx) const override;
    std::string GetKernelBody(TContext* ctx) const override;
};

class ElemwiseMultiTypeQS8 : public KernelFunc {
public:
    bool IsAvailable(TContext* ctx) const override;
    std::string GetKernelSymbol(TContext* ctx) const override;
    std::string GetKernelBody(TContext* ctx) const override;
};

class TypeCvtQS32QS8 : public KernelFunc {
public:
    bool IsAvailable(TContext* ctx) const override;
    std::string GetKernelSymbol(TContext* ctx) const override;
    std::string GetKernelBody(TContext* ctx) const override;
};

// qint8 x qint8 -> qint32 MatrixMul with the TypeCvt to qint8 that follows it folded in
// (attribute "fused_typecvt"), operand:0 A [M][K], operand:1 B [K][N] (a weight),
// operand:2 C [M][N] qint8. The reference has an int8 MatrixMul only for Arm
// (compiler/lib/KernelGen/Arm/Arm64/MatMulKernel/Int8DotMatMulM8N12K4.cpp:20-31); attribute
// names are those of BareMetal::MatrixMulKernel (compiler/lib/KernelGen/BareMetal/
// MatrixMul.cpp:13-43).
class MatMulQS8 : public KernelFunc {
public:
    bool IsAvailable(TContext* ctx) const override;
    std::string GetKernelSymbol(TContext* ctx) const override;
    std::string GetKernelBody(TContext* ctx) const override;
    std::string GetInitBody(TContext* ctx) const override;
};

// NCHW <-> NHWC at the model boundary
class RelayoutQS8 : public KernelFunc {
public:
    bool IsAvailable(TContext* ctx) const override;
    std::string GetKernelSymbol(TContext* ctx) const override;
    std::string GetKernelBody(TContext* ctx) const override;
};

struct ArchKernelPack {
    static std::vector<const KernelFunc*> GetKernel(KernelPack::KernType kernel_type);
};

// "#include" lines every generated stub starts with
std::string GenStubPrologue();

}  // namespace Cuda
}  // namespace KernelGen
}  // namespace megcc
