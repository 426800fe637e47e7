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

// Bytes of device scratch an operator needs, answered directly (the reference sizes
// workspaces by running the generated *_workspace function through a JIT at compile time,
// compiler/lib/Dialect/Kernel/Transforms/KernelTemplate.cpp:18-35). Kernels of this pack that
// need scratch derive from it.
class WithWorkspace {
public:
    virtual ~WithWorkspace() = default;
    virtual size_t WorkspaceBytes(TContext* ctx) const = 0;
};

// qint8 ConvBias, activations NHWC. Admits a subset of what BareMetal::ConvGeneral admits
// (compiler/lib/KernelGen/BareMetal/ConvKernel.cpp:16-46).
class ConvBiasQS8 : public KernelFunc, public WithWorkspace {
public:
    bool IsAvailable(TContext* ctx) const override;
    std::string GetKernelSymbol(TContext* ctx) const override;
    std::string GetKernelBody(TContext* ctx) const override;
    std::string GetInitBody(TContext* ctx) const override;
    std::string GetWorkspaceBody(TContext* ctx) const override;
    // bytes of device scratch the kernel needs for the operator `ctx` describes
    size_t WorkspaceBytes(TContext* ctx) const override;
};

// ---- fp32 path (the detector configuration and the fp32 MatrixMul sweep) ----

// fp32 ConvBias, activations NHWC. nonlineMode IDENTITY / RELU / SIGMOID / H_SWISH as the
// reference's fp32 kernels take it (compiler/lib/KernelGen/GeneralIntrinsic/ConvKernel/
// Fp32Im2col.cpp:122-156), plus SILU: the Elemwise kernel that follows the ConvBias in a
// YOLOX-style graph, folded into the epilogue. An optional z operand (attribute
// fuse_elemwise_mode = "ADD") is added after the activation (the bottleneck shortcut).
class ConvBiasF32 : public KernelFunc, public WithWorkspace {
public:
    bool IsAvailable(TContext* ctx) const override;
    std::string GetKernelSymbol(TContext* ctx) const override;
    std::string GetKernelBody(TContext* ctx) const override;
    std::string GetInitBody(TContext* ctx) const override;
    std::string GetWorkspaceBody(TContext* ctx) const override;
    size_t WorkspaceBytes(TContext* ctx) const override;
};

// C[M][N] = A[M][K] x B[K][N], all fp32, B a weight
// (compiler/lib/KernelGen/GeneralIntrinsic/MatMulKernel/Fp32MatMulM4N12.cpp:8-160)
class MatMulF32 : public KernelFunc, public WithWorkspace {
public:
    bool IsAvailable(TContext* ctx) const override;
    std::string GetKernelSymbol(TContext* ctx) const override;
    std::string GetKernelBody(TContext* ctx) const override;
    std::string GetInitBody(TContext* ctx) const override;
    std::string GetWorkspaceBody(TContext* ctx) const override;
    size_t WorkspaceBytes(TContext* ctx) const override;
};

// Elemwise fp32, same-shape operands (compiler/lib/KernelGen/BareMetal/ElemwiseKernel.cpp:413-431)
class ElemwiseF32 : public KernelFunc {
public:
    bool IsAvailable(TContext* ctx) const override;
    std::string GetKernelSymbol(TContext* ctx) const override;
    std::string GetKernelBody(TContext* ctx) const override;
};

// Concat along channels (compiler/lib/KernelGen/BareMetal/Concat.cpp:10-78, axis 1); with the
// attribute "focus" the single NCHW input is read through its four stride-2 slices
class ConcatF32 : public KernelFunc {
public:
    bool IsAvailable(TContext* ctx) const override;
    std::string GetKernelSymbol(TContext* ctx) const override;
    std::string GetKernelBody(TContext* ctx) const override;
};

// Resize NEAREST fp32 (compiler/lib/KernelGen/BareMetal/Resize.cpp:13-33)
class ResizeF32 : public KernelFunc {
public:
    bool IsAvailable(TContext* ctx) const override;
    std::string GetKernelSymbol(TContext* ctx) const override;
    std::string GetKernelBody(TContext* ctx) const override;
};

// Pooling fp32 (compiler/lib/KernelGen/BareMetal/Pooling.cpp:15-29)
class PoolingF32 : public KernelFunc {
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
