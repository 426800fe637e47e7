/*
 * Runtime data structures that generated kernel stubs receive.
 *
 * Field order, types and enum values are the binary contract of the reference runtime
 * (runtime/src/tinynn.h:9-54, runtime/src/data_struct.h:12-59 and :131-153,
 * runtime/src/device.h:8-21): a stub compiled against this header can be linked into
 * the reference runtime and the other way round. Additions are only ever made at the
 * end of an enum or struct: the CUDA device kind, and a stream / device ordinal after
 * RuntimeOpt's existing member (the reference reserves RuntimeOpt "for expand later").
 */
#ifndef MEGCC_B200_RUNTIME_H_
#define MEGCC_B200_RUNTIME_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MAX_DIM (7)

typedef enum {
    TinyNN_SUCCESS = 0,
    TinyNN_ERROR_NULL_PTR = 1,
    TinyNN_ERROR_STANDER = 2,
    TinyNN_ERROR_RUNTIME = 3,
    TinyNN_ERROR_OUT_OF_RANGE = 4,
    TinyNN_ERROR_NO_FOUND = 5,
    TinyNN_ERROR_NO_IMPLEMENT = 6,
    TinyNN_ERROR_MODEL_PARSE = 7,
    TinyNN_ERROR_OPEN_FILE_ERROR = 8,
    TinyNN_ERROR_MEMORY_MALLOC = 9,
    TinyNN_ERROR_UNSUPPORTED_INSTRUCTION_TYPE = 10,
    TinyNN_ERROR_UNSUPPORTED_DTYPE_TYPE = 11,
    TinyNN_ERROR_INVALID_LAYOUT = 12,
    TinyNN_ERROR = 13,
} TinyNNStatus;

typedef enum {
    TinyNN_FLOAT = 0,
    TinyNN_FLOAT16 = 1,
    TinyNN_INT = 2,
    TinyNN_INT8 = 3,
    TinyNN_INT16 = 4,
    TinyNN_UINT8 = 5,
    TinyNN_QINT8 = 100,
    TinyNN_QINT32 = 101,
    TinyNN_QUINT8 = 102,
} TinyNNDType;

typedef enum {
    TinyNN_NCHW = 0,
    TinyNN_NHWC,
    TinyNN_NCHW4,
    TinyNN_NCHW8,
    TinyNN_OIHW,
} TinyNNFormat;

typedef enum {
    TinyNN_BARE_METAL = 0,
    TinyNN_ARM64,
    TinyNN_ARM32,
    TinyNN_ARM64_V82,
    TinyNN_ARM32_V82,
    TinyNN_OPENCL_MALI,
    TinyNN_WEB_ASSEMBLY,
    TinyNN_CUDA_SM100 /* added at the end */
} TinyNNDevice;

typedef struct {
    float scale;
    uint8_t zero_point;
} DTypeParam;

typedef struct {
    TinyNNDType type_enum;
    DTypeParam param;
} DType;

/* dims are logical (N, C, H, W for activations); stride is in elements and tells the
 * physical order, so an NHWC buffer has stride {H*W*C, 1, W*C, C} and format TinyNN_NHWC */
typedef struct {
    int nr_dim;
    uint32_t dims[MAX_DIM];
    int stride[MAX_DIM];
    TinyNNFormat format;
} Layout;

typedef struct Tensor {
    char* name;
    DType dtype;
    Layout layout;
    void* ptr; /* device memory for the CUDA device kind */
    size_t offset;
    int use_count;
    int is_weight;
    int is_dynamic;
    uint32_t checksum;
    size_t size;
    int is_shared;
    int is_input;
} Tensor;

typedef struct {
    void* ptr;
    size_t size;
    size_t offset;
} Workspace;

typedef struct {
    int alignment;
    TinyNNDevice device_type;
    void* (*malloc)(size_t length);
    void (*free)(void* ptr);
} Device;

typedef struct RuntimeOpt {
    const Device* device;
    /* ---- additions ---- */
    void* stream;  /* cudaStream_t every kernel of the model is issued on */
    int device_id; /* CUDA ordinal */
    /* the Opr being executed, for the runtime's own kernel implementations (one function
     * serves every symbol there); generated stubs have their attributes baked in and ignore it */
    const void* opr;
} RuntimeOpt;

static inline void* mb200_opt_stream(const RuntimeOpt* opt) {
    return opt ? opt->stream : (void*)0;
}

/* the four uniform function types of generated code */
typedef TinyNNStatus (*KernelFunc)(
        Tensor** inputs, int nr_input, Tensor** outputs, int nr_output,
        const Workspace* workspace, const RuntimeOpt* opt);
typedef TinyNNStatus (*InitFunc)(
        Tensor** inputs, int nr_input, Tensor* out_weights, int* nr_out_weight,
        const RuntimeOpt* opt);
typedef TinyNNStatus (*WorkspaceFunc)(
        Tensor** inputs, int nr_input, int nr_thread, size_t* workspace);
typedef TinyNNStatus (*DeduceFunc)(
        Tensor** inputs, int nr_input, Tensor** outputs, int nr_output);

#ifdef __cplusplus
}
#endif
#endif /* MEGCC_B200_RUNTIME_H_ */
