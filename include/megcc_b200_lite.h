/*
 * LITE_* C API of the megcc_b200 runtime (libmegcc_b200.so).
 *
 * Same names, argument order, struct layouts, enum values and status codes as the
 * reference runtime's lite-c interface (runtime/include/lite-c/common_enum_c.h,
 * tensor_c.h, network_c.h, global_c.h; implementation runtime/src/lite/network.c and
 * tensor.c), so a program written against the reference links against this library
 * unchanged. Only the functions the reference actually implements are provided, plus the
 * device getters/setters it declares but leaves unimplemented. Every function returns a
 * TinyNNStatus as int (0 = success).
 *
 * Behaviour that differs because the work happens on a GPU:
 *  - LITE_forward enqueues one CUDA-graph launch on the network's stream and returns;
 *    LITE_wait synchronises and reports a device-side error, if any. Reading an output
 *    with LITE_get_tensor_memory also waits, so code that never calls LITE_wait (legal
 *    with the reference, where it is a no-op: runtime/src/lite/network.c:229-232) still
 *    sees finished results.
 *  - a host pointer given to LITE_reset_tensor_memory is copied to the device inside
 *    LITE_forward; a device pointer is used in place. Outputs are returned in host
 *    memory unless the output was declared with LiteIO.is_host == 0 in LiteNetworkIO.
 *  - LiteConfig.device_id selects the CUDA ordinal (the reference ignores the config,
 *    runtime/src/lite/network.c:47-56).
 */
#ifndef MEGCC_B200_LITE_H_
#define MEGCC_B200_LITE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LITE_API __attribute__((visibility("default")))
#define LAYOUT_MAX_DIM (7)

typedef enum LiteLogLevel { LITE_DEBUG = 0, LITE_INFO = 1, LITE_WARN = 2, LITE_ERROR = 3 } LiteLogLevel;
typedef enum LiteBackend { LITE_DEFAULT = 0 } LiteBackend;
typedef enum LiteDeviceType {
    LITE_CPU = 0,
    LITE_CUDA = 1,
    LITE_ATLAS = 3,
    LITE_NPU = 4,
    LITE_DEVICE_DEFAULT = 5,
} LiteDeviceType;
typedef enum LiteDataType {
    LITE_FLOAT = 0,
    LITE_HALF = 1,
    LITE_INT = 2,
    LITE_INT16 = 3,
    LITE_INT8 = 4,
    LITE_UINT8 = 5,
    LITE_UINT = 6,
    LITE_UINT16 = 7,
    LITE_INT64 = 8,
} LiteCDataType;
typedef enum LiteTensorPhase { LITE_IO = 0, LITE_INPUT = 1, LITE_OUTPUT = 2 } LiteTensorPhase;
typedef enum LiteIOType { LITE_IO_VALUE = 0, LITE_IO_SHAPE = 1 } LiteIOType;

typedef struct LiteLayout {
    size_t shapes[LAYOUT_MAX_DIM];
    size_t ndim;
    LiteCDataType data_type;
} LiteLayout;

typedef struct Options {
    int weight_preprocess;
    int fuse_preprocess;
    int fake_next_exec;
    int var_sanity_check_first_run;
    int const_shape;
    int force_dynamic_alloc;
    int force_output_dynamic_alloc;
    int no_profiling_on_shape_change;
    int jit_level;
    int comp_node_seq_record_level;
    int graph_opt_level;
    int async_exec_level;
    int enable_nchw44;
    int enable_nchw44_dot;
    int enable_nchw88;
    int enable_nhwcd4;
    int enable_nchw4;
    int enable_nchw32;
    int enable_nchw64;
} LiteOptions;

typedef struct LiteConfig {
    int has_compression;
    int device_id;
    LiteDeviceType device_type;
    LiteBackend backend;
    const char* bare_model_cryption_name;
    LiteOptions options;
} LiteConfig;

typedef struct LiteIO {
    const char* name;
    int is_host;
    LiteIOType io_type;
    LiteLayout config_layout;
} LiteIO;

typedef struct LiteNetworkIO {
    LiteIO* inputs;
    LiteIO* outputs;
    size_t input_size;
    size_t output_size;
} LiteNetworkIO;

typedef void* LiteNetwork;
typedef void* LiteTensor;

/* runtime/src/lite/network.c:22-41 */
LITE_API LiteConfig* default_config(void);
LITE_API LiteNetworkIO* default_network_io(void);

/* runtime/src/lite/network.c:47-56 */
LITE_API int LITE_make_network(
        LiteNetwork* network, const LiteConfig config, const LiteNetworkIO network_io);
/* runtime/src/lite/network.c:58-65; the buffer is borrowed until the network is destroyed */
LITE_API int LITE_load_model_from_mem(LiteNetwork network, void* model_mem, size_t size);
/* runtime/src/lite/network.c:67-77 */
LITE_API int LITE_load_model_with_shared_mem(LiteNetwork network, void* model_mem, size_t size);
/* runtime/src/lite/network.c:79-101 */
LITE_API int LITE_load_model_from_path(LiteNetwork network, const char* model_path);
/* runtime/src/lite/network.c:103-159 */
LITE_API int LITE_get_io_tensor(
        LiteNetwork network, const char* io_name, LiteTensorPhase phase, LiteTensor* tensor);
/* runtime/src/lite/network.c:161-169 */
LITE_API int LITE_get_tensor_total_size_in_byte(const LiteTensor tensor, size_t* size);
/* runtime/src/lite/network.c:171-227 */
LITE_API int LITE_forward(const LiteNetwork network);
/* runtime/src/lite/network.c:229-232 */
LITE_API int LITE_wait(const LiteNetwork network);
/* runtime/src/lite/network.c:234-283 */
LITE_API int LITE_get_input_name(const LiteNetwork network, size_t index, const char** name);
LITE_API int LITE_get_output_name(const LiteNetwork network, size_t index, const char** name);
LITE_API int LITE_get_all_input_name(const LiteNetwork network, size_t* size, const char** name);
LITE_API int LITE_get_all_output_name(const LiteNetwork network, size_t* size, const char** name);
/* runtime/src/lite/network.c:285-303 (spelling of the symbol is the reference's) */
LITE_API int LITE_share_runtime_memroy(LiteNetwork src_network, LiteNetwork dst_network);
/* runtime/src/lite/network.c:305-368 */
LITE_API int LITE_destroy_network(LiteNetwork network);

/* runtime/src/lite/tensor.c:59-76 */
LITE_API int LITE_get_tensor_memory(const LiteTensor tensor, void** data);
/* runtime/src/lite/tensor.c:78-91 */
LITE_API int LITE_set_tensor_layout(LiteTensor tensor, const LiteLayout layout);
/* runtime/src/lite/tensor.c:93-112 */
LITE_API int LITE_reset_tensor_memory(
        LiteTensor tensor, void* prepared_data, size_t data_length_in_byte);
/* runtime/src/lite/tensor.c:114-134; fails for quantised tensors exactly like the reference */
LITE_API int LITE_get_tensor_layout(const LiteTensor tensor, LiteLayout* layout);
/* runtime/src/lite/tensor.c:136-139 */
LITE_API int LITE_destroy_tensor(LiteTensor tensor);

/* runtime/src/lite/global.c:6-14 */
LITE_API int LITE_set_log_level(LiteLogLevel level);
LITE_API int LITE_get_log_level(LiteLogLevel* level);
LITE_API const char* LITE_get_last_error(void);

/* declared by runtime/include/lite-c/network_c.h:330-378 and tensor_c.h, not implemented
 * by the reference; meaningful on a GPU */
LITE_API int LITE_get_device_id(const LiteNetwork network, int* device_id);
LITE_API int LITE_set_device_id(LiteNetwork network, int device_id);
LITE_API int LITE_get_device_type(const LiteNetwork network, LiteDeviceType* device_type);
LITE_API int LITE_get_tensor_device_type(const LiteTensor tensor, LiteDeviceType* device_type);

/* ---- additions; none of these has a counterpart in the reference ----
 * The CUDA stream (cudaStream_t) all work of the network is issued on, for callers that
 * time or order their own work against it. */
LITE_API int mb200_lite_stream(const LiteNetwork network, void** stream);
/* Registers the function tables of a generated kernels.c (what load_kernel_init_function
 * fills in the reference, compiler/lib/Target/TinyNN/KernelExporter.cpp:15-66) before a model
 * is loaded: kernels[kernel_id] and init_kernels[init_id] then execute the model's Oprs as
 * runtime/src/vm/op.c:161-163 and runtime/src/init.c:29-131 do. NULL entries, and ids beyond
 * the tables, fall to the library's own implementation of the Opr's symbol; an Opr whose
 * symbol the library does not know runs only through a registered entry. The function types
 * are those of include/megcc_b200_runtime.h (void* here to keep this header free of it). */
LITE_API int mb200_lite_set_kernel_tables(
        LiteNetwork network, const void* kernels, int nr_kernels, const void* init_kernels,
        int nr_init);
/* Per-network switches. "use_graph" (default 1): replay the instruction list as one CUDA
 * graph; 0 issues the kernels one by one on every forward. "profile": as
 * mb200_lite_set_profile. New networks take their defaults from the environment once per
 * process (MB200_NO_GRAPH=1, MB200_PROFILE=1); nothing reads the environment afterwards. */
LITE_API int mb200_lite_set_option(LiteNetwork network, const char* name, int value);
/* Per-instruction timing (the reference's compile-time TINYNN_PROFILE_KERNEL,
 * runtime/src/lite/network.c:187-224, as a run-time switch): while enabled every forward
 * runs instruction by instruction with a CUDA event pair around each one. */
LITE_API int mb200_lite_set_profile(LiteNetwork network, int enable);
/* one line per instruction: "<opr name> <kernel symbol> <mean ms> <samples>" */
LITE_API int mb200_lite_profile(const LiteNetwork network, char* out, size_t cap);

#ifdef __cplusplus
}
#endif
#endif /* MEGCC_B200_LITE_H_ */
