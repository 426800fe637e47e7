/* TEST INFRASTRUCTURE (checker only).
 *
 * The header MegCC's exporter generates next to a model
 * (compiler/lib/Target/TinyNN/KernelExporter.cpp:15-45), written by hand for
 * oracle/ref_lite_runner.c: the tables are sized generously and filled at run time from the
 * symbols the model's Oprs name, so that one pre-built runner serves any model whose
 * kernels oracle/_ref/libmegcc_ref_kernels.so holds. */
#ifndef KERNEL_H
#define KERNEL_H

#include "data_struct.h"
#include "stdint.h"
#include "string.h"

#define NR_KERNELS (1024)
#define NR_INIT (1024)
#define NR_DEDUCE_SHAPE (1)
#define NR_WORKSPACE (1024)

extern KernelFunc kernels[NR_KERNELS];
extern InitFunc init_kernels[NR_INIT];
extern WorkspaceFunc workspace_func[NR_WORKSPACE];
extern DeduceFunc deduce_func[NR_DEDUCE_SHAPE];

void load_kernel_init_function();

#endif
