/* TEST INFRASTRUCTURE (checker only): the instruction switch MegCC's exporter generates
 * (compiler/lib/Target/TinyNN/KernelExporter.cpp:113-124) for models that hold Opr and
 * MemForward instructions only. */
#define ENABLE_INST_OPR 1
#define ENABLE_INST_MEMFORWARD 1
