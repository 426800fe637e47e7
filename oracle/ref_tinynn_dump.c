/* TEST INFRASTRUCTURE (checker only).
 *
 * Reads a tinynn model with the REFERENCE's own flatcc-generated reader
 * (runtime/src/cheader/model_reader.h, the accessors runtime/src/parse.c:424-559 uses) and
 * prints what it sees, so a test can prove that a model written by megcc_b200 is the
 * same model to the reference's reader. Compiled against the reference headers where they
 * lie by oracle/Makefile; output binary oracle/_ref/ref_tinynn_dump.
 */
#include <stdio.h>
#include <stdlib.h>

#include "model_reader.h"

#undef ns
#define ns(x) FLATBUFFERS_WRAP_NAMESPACE(MegCC, x)

static void print_layout(ns(Layout_table_t) l) {
    flatbuffers_int32_vec_t dims = ns(Layout_dims(l));
    flatbuffers_int32_vec_t stride = ns(Layout_stride(l));
    size_t n = flatbuffers_int32_vec_len(dims);
    printf(" format=%d dims=", (int)ns(Layout_format(l)));
    for (size_t i = 0; i < n; ++i)
        printf("%d%s", flatbuffers_int32_vec_at(dims, i), i + 1 < n ? "x" : "");
    printf(" stride=");
    for (size_t i = 0; i < n; ++i)
        printf("%d%s", flatbuffers_int32_vec_at(stride, i), i + 1 < n ? "x" : "");
}

int main(int argc, char** argv) {
    if (argc != 2) {
        fprintf(stderr, "usage: %s model.tiny\n", argv[0]);
        return 2;
    }
    FILE* f = fopen(argv[1], "rb");
    if (!f)
        return 2;
    fseek(f, 0, SEEK_END);
    long size = ftell(f);
    fseek(f, 0, SEEK_SET);
    void* buf = aligned_alloc(64, (size + 63) / 64 * 64);
    if (fread(buf, 1, size, f) != (size_t)size)
        return 2;
    fclose(f);
    ns(Model_table_t) model = ns(Model_as_root(buf));
    if (!model) {
        printf("no root\n");
        return 1;
    }
    printf("model name=%s const_shape=%d\n", ns(Model_name(model)), (int)ns(Model_const_shape(model)));
    ns(Weight_vec_t) ws = ns(Model_weight_pool(model));
    for (size_t i = 0; i < ns(Weight_vec_len(ws)); ++i) {
        ns(Weight_table_t) w = ns(Weight_vec_at(ws, i));
        ns(DType_table_t) dt = ns(Weight_dtype(w));
        printf("weight %s dtype=%d scale=%.9g bytes=%zu", ns(Weight_name(w)), (int)ns(DType_type(dt)),
               ns(DTypeParam_scale(ns(DType_param(dt)))), flatbuffers_int8_vec_len(ns(Weight_data(w))));
        print_layout(ns(Weight_layout(w)));
        printf("\n");
    }
    ns(DeviceModel_vec_t) dms = ns(Model_device_models(model));
    for (size_t m = 0; m < ns(DeviceModel_vec_len(dms)); ++m) {
        ns(DeviceModel_table_t) dm = ns(DeviceModel_vec_at(dms, m));
        ns(Tensor_vec_t) ts = ns(DeviceModel_tensor_pool(dm));
        ns(Instruction_union_vec_t) insts = ns(DeviceModel_instructions_union(dm));
        printf("device_model %zu device=%d tensor_memory=%llu tensors=%zu instructions=%zu\n", m,
               (int)ns(DeviceModel_device(dm)), (unsigned long long)ns(DeviceModel_tensor_memory(dm)),
               ns(Tensor_vec_len(ts)), ns(Instruction_union_vec_len(insts)));
        for (size_t i = 0; i < ns(Tensor_vec_len(ts)); ++i) {
            ns(Tensor_table_t) t = ns(Tensor_vec_at(ts, i));
            ns(DType_table_t) dt = ns(Tensor_dtype(t));
            printf("tensor %s offset=%lld dtype=%d scale=%.9g", ns(Tensor_name(t)),
                   (long long)ns(Tensor_offset(t)), (int)ns(DType_type(dt)),
                   ns(DTypeParam_scale(ns(DType_param(dt)))));
            print_layout(ns(Tensor_layout(t)));
            printf("\n");
        }
        for (size_t i = 0; i < ns(Instruction_union_vec_len(insts)); ++i) {
            ns(Instruction_union_t) u = ns(Instruction_union_vec_at(insts, i));
            if (u.type != ns(Instruction_Opr)) {
                printf("instruction type=%d\n", (int)u.type);
                continue;
            }
            ns(Opr_table_t) o = (ns(Opr_table_t))u.value;
            flatbuffers_int32_vec_t in = ns(Opr_inputs(o));
            flatbuffers_int8_vec_t in_t = ns(Opr_input_types(o));
            flatbuffers_int32_vec_t out = ns(Opr_outputs(o));
            printf("opr %s kernel_id=%d init_id=%d deduce_id=%d ws=%lld in=", ns(Opr_type(o)),
                   ns(Opr_kernel_id(o)), ns(Opr_init_id(o)), ns(Opr_deduce_id(o)),
                   (long long)ns(Workspace_size(ns(Opr_workspace(o)))));
            for (size_t k = 0; k < flatbuffers_int32_vec_len(in); ++k)
                printf("%c%d,", flatbuffers_int8_vec_at(in_t, k) ? 'w' : 't',
                       flatbuffers_int32_vec_at(in, k));
            printf(" out=");
            for (size_t k = 0; k < flatbuffers_int32_vec_len(out); ++k)
                printf("%d,", flatbuffers_int32_vec_at(out, k));
            printf("\n");
        }
        flatbuffers_int32_vec_t ins = ns(DeviceModel_inputs(dm));
        flatbuffers_int32_vec_t outs = ns(DeviceModel_outputs(dm));
        for (size_t i = 0; i < flatbuffers_int32_vec_len(ins); ++i)
            printf("input %d\n", flatbuffers_int32_vec_at(ins, i));
        for (size_t i = 0; i < flatbuffers_int32_vec_len(outs); ++i)
            printf("output %d\n", flatbuffers_int32_vec_at(outs, i));
    }
    return 0;
}
