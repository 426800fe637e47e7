/* TEST INFRASTRUCTURE (checker and CPU baseline only; never linked into the product).
 *
 * The reference's own C runtime (runtime/src: parse.c, init.c, vm.c, vm/op.c, lite/network.c ...,
 * compiled unmodified from where they lie by oracle/Makefile) running the BARE_METAL
 * DeviceModel of a tinynn model through its own LITE_* API, with the reference's own generated
 * x86 kernels (oracle/_ref/libmegcc_ref_kernels.so). What MegCC generates per model
 * (kernels.h / kernels.c: the function tables indexed by kernel_id) is provided generically:
 * before the model is loaded, this program reads the Oprs' symbols with the reference's
 * flatcc reader and fills kernels[] / init_kernels[] / workspace_func[] by name.
 *
 *   ref_lite_runner model.tiny input.bin output.bin [iterations] [cpu]
 *
 * input.bin: raw bytes of the first input tensor; output.bin: raw bytes of the first output.
 * Prints "forward_ms <mean>" for the timed iterations (after one untimed forward), following
 * the flow of runtime/example/standard_OS/lite_main.c:281-404.
 */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <sched.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/time.h>

#include "kernels.h"
#include "lite-c/common_enum_c.h"
#include "lite-c/global_c.h"
#include "lite-c/network_c.h"
#include "lite-c/tensor_c.h"
#include "model_reader.h"

#undef ns
#define ns(x) FLATBUFFERS_WRAP_NAMESPACE(MegCC, x)

KernelFunc kernels[NR_KERNELS];
InitFunc init_kernels[NR_INIT];
WorkspaceFunc workspace_func[NR_WORKSPACE];
DeduceFunc deduce_func[NR_DEDUCE_SHAPE];

/* the tables are filled by main() before the runtime asks for them */
void load_kernel_init_function() {}

static TinyNNStatus no_init(
        Tensor** inputs, int nr_input, Tensor* out_weights, int* nr_out_weight,
        const RuntimeOpt* opt) {
    (void)inputs, (void)nr_input, (void)out_weights, (void)opt;
    if (nr_out_weight)
        *nr_out_weight = 0;
    return TinyNN_SUCCESS;
}

static void* read_file(const char* path, size_t* size) {
    FILE* f = fopen(path, "rb");
    if (!f)
        return NULL;
    fseek(f, 0, SEEK_END);
    *size = (size_t)ftell(f);
    fseek(f, 0, SEEK_SET);
    void* buf = aligned_alloc(64, (*size + 63) / 64 * 64);
    if (fread(buf, 1, *size, f) != *size) {
        fclose(f);
        return NULL;
    }
    fclose(f);
    return buf;
}

/* kernels[kernel_id] etc. for every Opr of the BARE_METAL DeviceModels */
static int fill_tables(void* model_buf, void* lib) {
    ns(Model_table_t) model = ns(Model_as_root(model_buf));
    if (!model)
        return -1;
    ns(DeviceModel_vec_t) dms = ns(Model_device_models(model));
    int found = 0;
    for (size_t m = 0; m < ns(DeviceModel_vec_len(dms)); ++m) {
        ns(DeviceModel_table_t) dm = ns(DeviceModel_vec_at(dms, m));
        if (ns(DeviceModel_device(dm)) != ns(Device_BARE_METAL))
            continue;
        ns(Instruction_union_vec_t) insts = ns(DeviceModel_instructions_union(dm));
        for (size_t i = 0; i < ns(Instruction_union_vec_len(insts)); ++i) {
            ns(Instruction_union_t) u = ns(Instruction_union_vec_at(insts, i));
            if (u.type != ns(Instruction_Opr))
                continue;
            ns(Opr_table_t) o = (ns(Opr_table_t))u.value;
            const char* sym = ns(Opr_type(o));
            const int kid = ns(Opr_kernel_id(o)), iid = ns(Opr_init_id(o)),
                      wid = ns(Opr_workspace_id(o));
            if (kid < 0 || kid >= NR_KERNELS || iid >= NR_INIT || wid >= NR_WORKSPACE) {
                fprintf(stderr, "kernel id out of range for %s\n", sym);
                return -1;
            }
            char name[600];
            kernels[kid] = (KernelFunc)dlsym(lib, sym);
            if (!kernels[kid]) {
                fprintf(stderr, "no reference kernel named %s\n", sym);
                return -1;
            }
            if (iid >= 0) {
                snprintf(name, sizeof(name), "%s_init", sym);
                InitFunc f = (InitFunc)dlsym(lib, name);
                init_kernels[iid] = f ? f : no_init;
            }
            if (wid >= 0) {
                snprintf(name, sizeof(name), "%s_workspace", sym);
                workspace_func[wid] = (WorkspaceFunc)dlsym(lib, name);
            }
            ++found;
        }
    }
    return found;
}

#define CHECK(call)                                                               \
    do {                                                                          \
        int rc_ = (call);                                                         \
        if (rc_ != 0) {                                                           \
            fprintf(stderr, "%s failed with status %d\n", #call, rc_);            \
            return 1;                                                             \
        }                                                                         \
    } while (0)

int main(int argc, char** argv) {
    if (argc < 4) {
        fprintf(stderr, "usage: %s model.tiny input.bin output.bin [iterations] [cpu]\n", argv[0]);
        return 2;
    }
    const int iterations = argc > 4 ? atoi(argv[4]) : 1;
    if (argc > 5) {
        cpu_set_t set;
        CPU_ZERO(&set);
        CPU_SET(atoi(argv[5]), &set);
        sched_setaffinity(0, sizeof(set), &set);
    }
    /* the kernel library lies beside this program */
    char lib_path[4096];
    Dl_info info;
    if (!dladdr((void*)&main, &info) || !info.dli_fname)
        return 2;
    snprintf(lib_path, sizeof(lib_path), "%s", info.dli_fname);
    char* slash = strrchr(lib_path, '/');
    snprintf(slash ? slash + 1 : lib_path, 64, "libmegcc_ref_kernels.so");
    void* lib = dlopen(lib_path, RTLD_NOW | RTLD_LOCAL);
    if (!lib) {
        fprintf(stderr, "cannot open %s: %s\n", lib_path, dlerror());
        return 2;
    }
    size_t model_size = 0, input_size = 0;
    void* model_buf = read_file(argv[1], &model_size);
    void* input = read_file(argv[2], &input_size);
    if (!model_buf || !input) {
        fprintf(stderr, "cannot read the model or the input\n");
        return 2;
    }
    const int n = fill_tables(model_buf, lib);
    if (n <= 0) {
        fprintf(stderr, "the model holds no BARE_METAL DeviceModel this runner can serve\n");
        return 3;
    }

    LiteNetwork net;
    CHECK(LITE_make_network(&net, *default_config(), *default_network_io()));
    CHECK(LITE_load_model_from_mem(net, model_buf, model_size));
    size_t nr_in = 0, nr_out = 0;
    CHECK(LITE_get_all_input_name(net, &nr_in, NULL));
    CHECK(LITE_get_all_output_name(net, &nr_out, NULL));
    const char* in_names[16];
    const char* out_names[16];
    if (nr_in < 1 || nr_in > 16 || nr_out < 1 || nr_out > 16)
        return 3;
    CHECK(LITE_get_all_input_name(net, NULL, in_names));
    CHECK(LITE_get_all_output_name(net, NULL, out_names));
    LiteTensor in, out;
    CHECK(LITE_get_io_tensor(net, in_names[0], LITE_INPUT, &in));
    size_t need = 0;
    CHECK(LITE_get_tensor_total_size_in_byte(in, &need));
    if (need != input_size) {
        fprintf(stderr, "input holds %zu bytes, the model wants %zu\n", input_size, need);
        return 3;
    }
    CHECK(LITE_reset_tensor_memory(in, input, input_size));
    CHECK(LITE_forward(net));
    CHECK(LITE_wait(net));
    struct timeval t0, t1;
    gettimeofday(&t0, NULL);
    for (int i = 0; i < iterations; ++i) {
        CHECK(LITE_forward(net));
        CHECK(LITE_wait(net));
    }
    gettimeofday(&t1, NULL);
    CHECK(LITE_get_io_tensor(net, out_names[0], LITE_OUTPUT, &out));
    void* out_ptr = NULL;
    size_t out_size = 0;
    CHECK(LITE_get_tensor_memory(out, &out_ptr));
    CHECK(LITE_get_tensor_total_size_in_byte(out, &out_size));
    FILE* f = fopen(argv[3], "wb");
    if (!f || fwrite(out_ptr, 1, out_size, f) != out_size)
        return 2;
    fclose(f);
    if (iterations > 0)
        printf("forward_ms %.4f\n",
               ((t1.tv_sec - t0.tv_sec) * 1e3 + (t1.tv_usec - t0.tv_usec) * 1e-3) / iterations);
    printf("kernels %d output_bytes %zu\n", n, out_size);
    CHECK(LITE_destroy_network(net));
    return 0;
}
