/* TEST INFRASTRUCTURE (checker only; never linked into or called by the product).
 *
 * Plain-pointer door into the reference's own generated x86 kernels. It is
 * compiled against the reference runtime headers where they lie (the Tensor /
 * Layout / DType structs of runtime/src/data_struct.h:12-53) and linked into
 * oracle/_ref/libmegcc_ref_kernels.so together with the emitted kernel C files.
 * The generated kernels all have the uniform signature of
 * runtime/src/data_struct.h:131-133.
 */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "data_struct.h"

static int ref_log(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    int r = vfprintf(stderr, fmt, ap);
    va_end(ap);
    return r;
}
/* the generated code's TINYNN_ASSERT needs these two (runtime/src/utils.h:9-11) */
tinynn_log __tinynn_log__ = ref_log;
LiteLogLevel g_log_level = LITE_WARN;

typedef struct {
    void* ptr;
    int dtype; /* TinyNNDType value: 0 f32, 2 i32, 3 i8, 100 qsi8, 101 qsi32 */
    float scale;
    int ndim;
    int dims[MAX_DIM];
} RefOperand;

static void fill(Tensor* t, const RefOperand* o) {
    memset(t, 0, sizeof(*t));
    t->name = (char*)"t";
    t->dtype.type_enum = (TinyNNDType)o->dtype;
    t->dtype.param.scale = o->scale;
    t->layout.nr_dim = o->ndim;
    int stride = 1;
    for (int i = o->ndim - 1; i >= 0; --i) {
        t->layout.dims[i] = (uint32_t)o->dims[i];
        t->layout.stride[i] = stride;
        stride *= o->dims[i];
    }
    t->layout.format = TinyNN_NCHW;
    t->ptr = o->ptr;
}

static void* self_handle(void) {
    static void* h = NULL;
    if (!h) {
        Dl_info info;
        if (dladdr((void*)&self_handle, &info) && info.dli_fname)
            h = dlopen(info.dli_fname, RTLD_NOW | RTLD_LOCAL);
    }
    return h;
}

int megcc_ref_has(const char* symbol) {
    void* h = self_handle();
    return h && dlsym(h, symbol) != NULL;
}

/* returns the kernel's TinyNNStatus, or -1 when the symbol was not pre-built.
 * Follows the reference's own test harness (compiler/test/kernel/common/src/cc_proxy.cpp
 * :125-255): <symbol>_workspace sizes the scratch, <symbol>_init preprocesses weights in its
 * three phases (count, describe, fill) and the processed weight replaces the input of the
 * same name, then the kernel runs. */
int megcc_ref_call(
        const char* symbol, const RefOperand* ins, int n_in, const RefOperand* outs,
        int n_out) {
    void* h = self_handle();
    if (!h)
        return -1;
    KernelFunc fn = (KernelFunc)dlsym(h, symbol);
    if (!fn)
        return -1;
    Tensor tin[8], tout[4];
    Tensor* pin[8];
    Tensor* pout[4];
    static char names[8][8] = {"in0", "in1", "in2", "in3", "in4", "in5", "in6", "in7"};
    if (n_in > 8 || n_out > 4)
        return -2;
    for (int i = 0; i < n_in; ++i) {
        fill(&tin[i], &ins[i]);
        tin[i].name = names[i];
        pin[i] = &tin[i];
    }
    for (int i = 0; i < n_out; ++i) {
        fill(&tout[i], &outs[i]);
        pout[i] = &tout[i];
    }
    char sym2[512];
    size_t ws_bytes = 0;
    snprintf(sym2, sizeof(sym2), "%s_workspace", symbol);
    WorkspaceFunc wfn = (WorkspaceFunc)dlsym(h, sym2);
    if (wfn && wfn(pin, n_in, 1, &ws_bytes) != TinyNN_SUCCESS)
        return -3;
    void* processed = NULL;
    Tensor new_weight;
    snprintf(sym2, sizeof(sym2), "%s_init", symbol);
    InitFunc ifn = (InitFunc)dlsym(h, sym2);
    if (ifn) {
        int count = 0;
        if (ifn(pin, n_in, NULL, &count, NULL) != TinyNN_SUCCESS || count > 1)
            return -4;
        if (count == 1) {
            memset(&new_weight, 0, sizeof(new_weight));
            if (ifn(pin, n_in, &new_weight, NULL, NULL) != TinyNN_SUCCESS)
                return -4;
            size_t bytes = new_weight.dtype.type_enum == TinyNN_FLOAT ? 4 : 1;
            for (int d = 0; d < new_weight.layout.nr_dim; ++d)
                bytes *= new_weight.layout.dims[d];
            processed = malloc(bytes + 64);
            new_weight.ptr = processed;
            if (ifn(pin, n_in, &new_weight, &count, NULL) != TinyNN_SUCCESS) {
                free(processed);
                return -4;
            }
            for (int i = 0; i < n_in; ++i)
                if (tin[i].name == new_weight.name)
                    tin[i] = new_weight;
        }
    }
    void* ws_mem = ws_bytes ? malloc(ws_bytes + 64) : NULL;
    Workspace ws = {ws_mem, ws_bytes, 0};
    RuntimeOpt opt = {NULL};
    const int rc = (int)fn(pin, n_in, pout, n_out, &ws, &opt);
    free(ws_mem);
    free(processed);
    return rc;
}
