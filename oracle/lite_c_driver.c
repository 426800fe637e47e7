/* TEST INFRASTRUCTURE. A C program written against the REFERENCE's own public headers
 * (runtime/include/lite-c/{global_c,network_c,tensor_c}.h; the Makefile compiles it with -I
 * pointing into the reference tree, nothing is copied) and linked against libmegcc_b200.so:
 * the flow of the reference's runtime/example/standard_OS/lite_main.c:281-404, reduced to one
 * input and one output. It proves that a user of the reference's C API can switch libraries
 * without touching source.
 *
 *   lite_c_driver <model.tiny> <input.bin> <output.bin> [forwards]
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "lite-c/global_c.h"
#include "lite-c/network_c.h"
#include "lite-c/tensor_c.h"

#define CHECK(call)                                              \
    do {                                                         \
        int rc_ = (call);                                        \
        if (rc_ != 0) {                                          \
            fprintf(stderr, "%s failed with status %d\n", #call, rc_); \
            return 1;                                            \
        }                                                        \
    } while (0)

static void* read_file(const char* path, size_t* size) {
    FILE* f = fopen(path, "rb");
    if (!f)
        return NULL;
    fseek(f, 0, SEEK_END);
    long n = ftell(f);
    fseek(f, 0, SEEK_SET);
    void* p = malloc(n > 0 ? (size_t)n : 1);
    if (p && fread(p, 1, (size_t)n, f) != (size_t)n) {
        free(p);
        p = NULL;
    }
    fclose(f);
    *size = (size_t)n;
    return p;
}

int main(int argc, char** argv) {
    if (argc < 4) {
        fprintf(stderr, "usage: %s model input output [forwards]\n", argv[0]);
        return 2;
    }
    const int forwards = argc > 4 ? atoi(argv[4]) : 1;
    LiteNetwork model;
    CHECK(LITE_make_network(&model, *default_config(), *default_network_io()));
    CHECK(LITE_load_model_from_path(model, argv[1]));

    size_t nr_input = 0, nr_output = 0;
    CHECK(LITE_get_all_input_name(model, &nr_input, NULL));
    CHECK(LITE_get_all_output_name(model, &nr_output, NULL));
    if (nr_input != 1 || nr_output != 1) {
        fprintf(stderr, "this driver takes models with one input and one output\n");
        return 1;
    }
    const char* in_name = NULL;
    const char* out_name = NULL;
    CHECK(LITE_get_all_input_name(model, NULL, &in_name));
    CHECK(LITE_get_all_output_name(model, NULL, &out_name));

    LiteTensor input, output;
    CHECK(LITE_get_io_tensor(model, in_name, LITE_INPUT, &input));
    size_t in_bytes = 0, file_bytes = 0;
    CHECK(LITE_get_tensor_total_size_in_byte(input, &in_bytes));
    void* data = read_file(argv[2], &file_bytes);
    if (!data || file_bytes != in_bytes) {
        fprintf(stderr, "input file holds %zu bytes, the model wants %zu\n", file_bytes, in_bytes);
        return 1;
    }
    CHECK(LITE_reset_tensor_memory(input, data, in_bytes));
    for (int i = 0; i < forwards; ++i) {
        CHECK(LITE_forward(model));
        CHECK(LITE_wait(model));
    }
    CHECK(LITE_get_io_tensor(model, out_name, LITE_OUTPUT, &output));
    void* out_ptr = NULL;
    size_t out_bytes = 0;
    CHECK(LITE_get_tensor_memory(output, &out_ptr));
    CHECK(LITE_get_tensor_total_size_in_byte(output, &out_bytes));
    FILE* f = fopen(argv[3], "wb");
    if (!f || fwrite(out_ptr, 1, out_bytes, f) != out_bytes) {
        fprintf(stderr, "cannot write %s\n", argv[3]);
        return 1;
    }
    fclose(f);
    printf("%s -> %s: %zu bytes in, %zu bytes out, %d forward(s)\n", in_name, out_name, in_bytes,
           out_bytes, forwards);
    CHECK(LITE_destroy_network(model));
    free(data);
    return 0;
}
