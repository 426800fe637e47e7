// TEST INFRASTRUCTURE (checker only).
//
// Builds the compile side of megcc_b200 INSIDE the reference's KernelGen: the CUDA kernel
// pack and the graph compiler are compiled with -DMEGCC_B200_IN_MEGCC_TREE against the
// reference's own KernelGen.h / TContext.h and linked with the reference's KernelGen objects
// (oracle/Makefile). It compiles a small network and writes the tinynn bytes to the file
// given on the command line; a test compares them with the stand-alone build's bytes, and
// checks that the reference's own registry still resolves the x86 kernel for the same
// operator, i.e. that both kernel packs live in one program.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "../include/megcc_b200_compiler.h"
#include "compiler/KernelGen/KernelGen.h"

int main(int argc, char** argv) {
    if (argc != 2)
        return 2;
    mb200c_graph* g = mb200c_graph_create("intree");
    const int x = mb200c_add_input(g, "data", 3, 64, 64, 0.02f);
    std::vector<int8_t> f1(64 * 3 * 7 * 7), f2(64 * 64 * 9);
    std::vector<int32_t> b(64);
    for (size_t i = 0; i < f1.size(); ++i)
        f1[i] = (int8_t)((i * 37) % 255 - 127);
    for (size_t i = 0; i < f2.size(); ++i)
        f2[i] = (int8_t)((i * 53) % 255 - 127);
    for (size_t i = 0; i < b.size(); ++i)
        b[i] = (int32_t)(i * 17) - 500;
    int y = mb200c_add_conv_bias(g, "stem", x, 64, 7, 7, 2, 3, 1, "RELU", f1.data(), 0.01f, b.data(),
                                 nullptr, 0.5f);
    y = mb200c_add_pooling(g, "pool", y, "MAX", 3, 2, 1);
    int z = mb200c_add_conv_bias(g, "conv", y, 64, 3, 3, 1, 1, 1, "IDENTITY", f2.data(), 0.01f,
                                 b.data(), nullptr, 2.0f);
    z = mb200c_add_qelemwise(g, "add", "QFUSE_ADD_RELU", z, y, 2.0f);
    if (x < 0 || y < 0 || z < 0 || mb200c_mark_output(g, z) < 0) {
        fprintf(stderr, "%s\n", mb200c_last_error());
        return 1;
    }
    const int batches[2] = {1, 32};
    const uint8_t* bytes = nullptr;
    size_t len = 0;
    if (mb200c_compile(g, batches, 2, &bytes, &len) < 0) {
        fprintf(stderr, "%s\n", mb200c_last_error());
        return 1;
    }
    FILE* f = fopen(argv[1], "wb");
    if (!f || fwrite(bytes, 1, len, f) != len)
        return 1;
    fclose(f);
    printf("%s", mb200c_kernel_symbols(g));
    // the reference's registry, in the same program
    auto kerns = megcc::KernelGen::KernelPack::GetKernel(
                         megcc::KernelGen::KernelPack::KernType::PoolingKernel,
                         megcc::KernelGen::Arch::BAREMETAL)
                         .first;
    printf("reference_pooling_candidates %zu\n", kerns.size());
    mb200c_graph_destroy(g);
    return 0;
}
