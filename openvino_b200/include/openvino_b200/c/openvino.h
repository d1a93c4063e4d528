/* C API of the inference runtime.
 *
 * The names, status codes, structs and calling conventions follow the reference C API
 * (src/bindings/c/include/openvino/c/ov_core.h, ov_model.h, ov_compiled_model.h, ov_infer_request.h,
 * ov_tensor.h, ov_shape.h, ov_partial_shape.h, ov_node.h, ov_prepostprocess.h), so that C programs written
 * against it compile and link against this library unchanged. Objects are opaque handles that the caller
 * releases with the matching *_free function; strings returned through char** are released with ov_free.
 * The library links the native core only (graph, IR reader/writer, passes, CPU executor, request state
 * machine): devices available through it are "CPU" and the policy names that resolve to it.
 */
#ifndef OPENVINO_B200_C_API_H
#define OPENVINO_B200_C_API_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OPENVINO_C_API(...) __attribute__((visibility("default"))) __VA_ARGS__

typedef enum {
    OK = 0,
    GENERAL_ERROR = -1,
    NOT_IMPLEMENTED = -2,
    NETWORK_NOT_LOADED = -3,
    PARAMETER_MISMATCH = -4,
    NOT_FOUND = -5,
    OUT_OF_BOUNDS = -6,
    UNEXPECTED = -7,
    REQUEST_BUSY = -8,
    RESULT_NOT_READY = -9,
    NOT_ALLOCATED = -10,
    INFER_NOT_STARTED = -11,
    NETWORK_NOT_READ = -12,
    INFER_CANCELLED = -13,
    INVALID_C_PARAM = -14,
    UNKNOWN_C_ERROR = -15,
    NOT_IMPLEMENT_C_METHOD = -16,
    UNKNOW_EXCEPTION = -17,
} ov_status_e;

typedef enum {
    DYNAMIC = 0U, BOOLEAN, BF16, F16, F32, F64, I4, I8, I16, I32, I64, U1, U2, U3, U4, U6, U8, U16, U32, U64, NF4,
    F8E4M3, F8E5M3, STRING, F4E2M1, F8E8M0,
} ov_element_type_e;

typedef struct { int64_t rank; int64_t* dims; } ov_shape_t;
typedef struct ov_dimension { int64_t min; int64_t max; } ov_dimension_t;
typedef ov_dimension_t ov_rank_t;
typedef struct ov_partial_shape { ov_rank_t rank; ov_dimension_t* dims; } ov_partial_shape_t;

typedef struct ov_core ov_core_t;
typedef struct ov_model ov_model_t;
typedef struct ov_compiled_model ov_compiled_model_t;
typedef struct ov_infer_request ov_infer_request_t;
typedef struct ov_tensor ov_tensor_t;
typedef struct ov_output_const_port ov_output_const_port_t;
typedef struct ov_output_port ov_output_port_t;
typedef struct ov_preprocess_prepostprocessor ov_preprocess_prepostprocessor_t;

typedef struct ov_version { const char* buildNumber; const char* description; } ov_version_t;
typedef struct { const char* device_name; ov_version_t version; } ov_core_version_t;
typedef struct { ov_core_version_t* versions; size_t size; } ov_core_version_list_t;
typedef struct { char** devices; size_t size; } ov_available_devices_t;
typedef struct { void (*callback_func)(void* args); void* args; } ov_callback_t;
typedef struct {
    enum Status { NOT_RUN, OPTIMIZED_OUT, EXECUTED } status;
    int64_t real_time;
    int64_t cpu_time;
    const char* node_name;
    const char* exec_type;
    const char* node_type;
} ov_profiling_info_t;
typedef struct { ov_profiling_info_t* profiling_infos; size_t size; } ov_profiling_info_list_t;

/* ---- common */
OPENVINO_C_API(const char*) ov_get_error_info(ov_status_e status);
OPENVINO_C_API(const char*) ov_get_last_err_msg(void);
OPENVINO_C_API(void) ov_free(const char* content);
OPENVINO_C_API(ov_status_e) ov_get_openvino_version(ov_version_t* version);
OPENVINO_C_API(void) ov_version_free(ov_version_t* version);
OPENVINO_C_API(void) ov_shutdown(void);

/* ---- shapes */
OPENVINO_C_API(ov_status_e) ov_shape_create(const int64_t rank, const int64_t* dims, ov_shape_t* shape);
OPENVINO_C_API(ov_status_e) ov_shape_free(ov_shape_t* shape);
OPENVINO_C_API(bool) ov_dimension_is_dynamic(const ov_dimension_t dim);
OPENVINO_C_API(bool) ov_rank_is_dynamic(const ov_rank_t rank);
OPENVINO_C_API(ov_status_e) ov_partial_shape_create(const int64_t rank, const ov_dimension_t* dims, ov_partial_shape_t* partial_shape_obj);
OPENVINO_C_API(ov_status_e) ov_partial_shape_create_dynamic(const ov_rank_t rank, const ov_dimension_t* dims, ov_partial_shape_t* partial_shape_obj);
OPENVINO_C_API(ov_status_e) ov_partial_shape_create_static(const int64_t rank, const int64_t* dims, ov_partial_shape_t* partial_shape_obj);
OPENVINO_C_API(void) ov_partial_shape_free(ov_partial_shape_t* partial_shape);
OPENVINO_C_API(ov_status_e) ov_partial_shape_to_shape(const ov_partial_shape_t partial_shape, ov_shape_t* shape);
OPENVINO_C_API(ov_status_e) ov_shape_to_partial_shape(const ov_shape_t shape, ov_partial_shape_t* partial_shape);
OPENVINO_C_API(bool) ov_partial_shape_is_dynamic(const ov_partial_shape_t partial_shape);
OPENVINO_C_API(const char*) ov_partial_shape_to_string(const ov_partial_shape_t partial_shape);

/* ---- core */
OPENVINO_C_API(ov_status_e) ov_core_create(ov_core_t** core);
OPENVINO_C_API(ov_status_e) ov_core_create_with_config(const char* xml_config_file, ov_core_t** core);
OPENVINO_C_API(void) ov_core_free(ov_core_t* core);
OPENVINO_C_API(ov_status_e) ov_core_read_model(const ov_core_t* core, const char* model_path, const char* bin_path, ov_model_t** model);
OPENVINO_C_API(ov_status_e) ov_core_read_model_from_memory_buffer(const ov_core_t* core, const char* model_str, const size_t str_len,
                                                                  const ov_tensor_t* weights, ov_model_t** model);
OPENVINO_C_API(ov_status_e) ov_core_compile_model(const ov_core_t* core, const ov_model_t* model, const char* device_name,
                                                  const size_t property_args_size, ov_compiled_model_t** compiled_model, ...);
OPENVINO_C_API(ov_status_e) ov_core_compile_model_from_file(const ov_core_t* core, const char* model_path, const char* device_name,
                                                            const size_t property_args_size, ov_compiled_model_t** compiled_model, ...);
OPENVINO_C_API(ov_status_e) ov_core_set_property(const ov_core_t* core, const char* device_name, ...);
OPENVINO_C_API(ov_status_e) ov_core_get_property(const ov_core_t* core, const char* device_name, const char* property_key, char** property_value);
OPENVINO_C_API(ov_status_e) ov_core_get_available_devices(const ov_core_t* core, ov_available_devices_t* devices);
OPENVINO_C_API(void) ov_available_devices_free(ov_available_devices_t* devices);
OPENVINO_C_API(ov_status_e) ov_core_import_model(const ov_core_t* core, const char* content, const size_t content_size, const char* device_name,
                                                 ov_compiled_model_t** compiled_model);
OPENVINO_C_API(ov_status_e) ov_core_get_versions_by_device_name(const ov_core_t* core, const char* device_name, ov_core_version_list_t* versions);
OPENVINO_C_API(void) ov_core_versions_free(ov_core_version_list_t* versions);

/* ---- model and ports */
OPENVINO_C_API(void) ov_model_free(ov_model_t* model);
OPENVINO_C_API(ov_status_e) ov_model_const_input(const ov_model_t* model, ov_output_const_port_t** input_port);
OPENVINO_C_API(ov_status_e) ov_model_const_input_by_name(const ov_model_t* model, const char* tensor_name, ov_output_const_port_t** input_port);
OPENVINO_C_API(ov_status_e) ov_model_const_input_by_index(const ov_model_t* model, const size_t index, ov_output_const_port_t** input_port);
OPENVINO_C_API(ov_status_e) ov_model_input(const ov_model_t* model, ov_output_port_t** input_port);
OPENVINO_C_API(ov_status_e) ov_model_input_by_name(const ov_model_t* model, const char* tensor_name, ov_output_port_t** input_port);
OPENVINO_C_API(ov_status_e) ov_model_input_by_index(const ov_model_t* model, const size_t index, ov_output_port_t** input_port);
OPENVINO_C_API(ov_status_e) ov_model_const_output(const ov_model_t* model, ov_output_const_port_t** output_port);
OPENVINO_C_API(ov_status_e) ov_model_const_output_by_index(const ov_model_t* model, const size_t index, ov_output_const_port_t** output_port);
OPENVINO_C_API(ov_status_e) ov_model_const_output_by_name(const ov_model_t* model, const char* tensor_name, ov_output_const_port_t** output_port);
OPENVINO_C_API(ov_status_e) ov_model_output(const ov_model_t* model, ov_output_port_t** output_port);
OPENVINO_C_API(ov_status_e) ov_model_output_by_index(const ov_model_t* model, const size_t index, ov_output_port_t** output_port);
OPENVINO_C_API(ov_status_e) ov_model_output_by_name(const ov_model_t* model, const char* tensor_name, ov_output_port_t** output_port);
OPENVINO_C_API(ov_status_e) ov_model_inputs_size(const ov_model_t* model, size_t* input_size);
OPENVINO_C_API(ov_status_e) ov_model_outputs_size(const ov_model_t* model, size_t* output_size);
OPENVINO_C_API(bool) ov_model_is_dynamic(const ov_model_t* model);
OPENVINO_C_API(ov_status_e) ov_model_reshape(const ov_model_t* model, const char** tensor_names, const ov_partial_shape_t* partial_shapes, size_t size);
OPENVINO_C_API(ov_status_e) ov_model_reshape_input_by_name(const ov_model_t* model, const char* tensor_name, const ov_partial_shape_t partial_shape);
OPENVINO_C_API(ov_status_e) ov_model_reshape_single_input(const ov_model_t* model, const ov_partial_shape_t partial_shape);
OPENVINO_C_API(ov_status_e) ov_model_reshape_by_port_indexes(const ov_model_t* model, const size_t* port_indexes, const ov_partial_shape_t* partial_shape,
                                                             size_t size);
OPENVINO_C_API(ov_status_e) ov_model_get_friendly_name(const ov_model_t* model, char** friendly_name);
OPENVINO_C_API(ov_status_e) ov_model_save(const ov_model_t* model, const char* xml_path, bool compress_to_fp16);

OPENVINO_C_API(ov_status_e) ov_const_port_get_shape(const ov_output_const_port_t* port, ov_shape_t* tensor_shape);
OPENVINO_C_API(ov_status_e) ov_port_get_shape(const ov_output_port_t* port, ov_shape_t* tensor_shape);
OPENVINO_C_API(ov_status_e) ov_port_get_any_name(const ov_output_const_port_t* port, char** tensor_name);
OPENVINO_C_API(ov_status_e) ov_port_get_partial_shape(const ov_output_const_port_t* port, ov_partial_shape_t* partial_shape);
OPENVINO_C_API(ov_status_e) ov_port_get_element_type(const ov_output_const_port_t* port, ov_element_type_e* tensor_type);
OPENVINO_C_API(void) ov_output_port_free(ov_output_port_t* port);
OPENVINO_C_API(void) ov_output_const_port_free(ov_output_const_port_t* port);

/* ---- compiled model */
OPENVINO_C_API(ov_status_e) ov_compiled_model_inputs_size(const ov_compiled_model_t* compiled_model, size_t* size);
OPENVINO_C_API(ov_status_e) ov_compiled_model_input(const ov_compiled_model_t* compiled_model, ov_output_const_port_t** input_port);
OPENVINO_C_API(ov_status_e) ov_compiled_model_input_by_index(const ov_compiled_model_t* compiled_model, const size_t index, ov_output_const_port_t** input_port);
OPENVINO_C_API(ov_status_e) ov_compiled_model_input_by_name(const ov_compiled_model_t* compiled_model, const char* name, ov_output_const_port_t** input_port);
OPENVINO_C_API(ov_status_e) ov_compiled_model_outputs_size(const ov_compiled_model_t* compiled_model, size_t* size);
OPENVINO_C_API(ov_status_e) ov_compiled_model_output(const ov_compiled_model_t* compiled_model, ov_output_const_port_t** output_port);
OPENVINO_C_API(ov_status_e) ov_compiled_model_output_by_index(const ov_compiled_model_t* compiled_model, const size_t index, ov_output_const_port_t** output_port);
OPENVINO_C_API(ov_status_e) ov_compiled_model_output_by_name(const ov_compiled_model_t* compiled_model, const char* name, ov_output_const_port_t** output_port);
OPENVINO_C_API(ov_status_e) ov_compiled_model_get_runtime_model(const ov_compiled_model_t* compiled_model, ov_model_t** model);
OPENVINO_C_API(ov_status_e) ov_compiled_model_create_infer_request(const ov_compiled_model_t* compiled_model, ov_infer_request_t** infer_request);
OPENVINO_C_API(ov_status_e) ov_compiled_model_set_property(const ov_compiled_model_t* compiled_model, ...);
OPENVINO_C_API(ov_status_e) ov_compiled_model_get_property(const ov_compiled_model_t* compiled_model, const char* property_key, char** property_value);
OPENVINO_C_API(ov_status_e) ov_compiled_model_export_model(const ov_compiled_model_t* compiled_model, const char* export_model_path);
OPENVINO_C_API(void) ov_compiled_model_free(ov_compiled_model_t* compiled_model);

/* ---- infer request */
OPENVINO_C_API(ov_status_e) ov_infer_request_set_tensor(ov_infer_request_t* infer_request, const char* tensor_name, const ov_tensor_t* tensor);
OPENVINO_C_API(ov_status_e) ov_infer_request_set_tensor_by_const_port(ov_infer_request_t* infer_request, const ov_output_const_port_t* port, const ov_tensor_t* tensor);
OPENVINO_C_API(ov_status_e) ov_infer_request_set_input_tensor_by_index(ov_infer_request_t* infer_request, const size_t idx, const ov_tensor_t* tensor);
OPENVINO_C_API(ov_status_e) ov_infer_request_set_input_tensor(ov_infer_request_t* infer_request, const ov_tensor_t* tensor);
OPENVINO_C_API(ov_status_e) ov_infer_request_set_output_tensor_by_index(ov_infer_request_t* infer_request, const size_t idx, const ov_tensor_t* tensor);
OPENVINO_C_API(ov_status_e) ov_infer_request_set_output_tensor(ov_infer_request_t* infer_request, const ov_tensor_t* tensor);
OPENVINO_C_API(ov_status_e) ov_infer_request_get_tensor(const ov_infer_request_t* infer_request, const char* tensor_name, ov_tensor_t** tensor);
OPENVINO_C_API(ov_status_e) ov_infer_request_get_tensor_by_const_port(const ov_infer_request_t* infer_request, const ov_output_const_port_t* port, ov_tensor_t** tensor);
OPENVINO_C_API(ov_status_e) ov_infer_request_get_input_tensor_by_index(const ov_infer_request_t* infer_request, const size_t idx, ov_tensor_t** tensor);
OPENVINO_C_API(ov_status_e) ov_infer_request_get_input_tensor(const ov_infer_request_t* infer_request, ov_tensor_t** tensor);
OPENVINO_C_API(ov_status_e) ov_infer_request_get_output_tensor_by_index(const ov_infer_request_t* infer_request, const size_t idx, ov_tensor_t** tensor);
OPENVINO_C_API(ov_status_e) ov_infer_request_get_output_tensor(const ov_infer_request_t* infer_request, ov_tensor_t** tensor);
OPENVINO_C_API(ov_status_e) ov_infer_request_infer(ov_infer_request_t* infer_request);
OPENVINO_C_API(ov_status_e) ov_infer_request_cancel(ov_infer_request_t* infer_request);
OPENVINO_C_API(ov_status_e) ov_infer_request_start_async(ov_infer_request_t* infer_request);
OPENVINO_C_API(ov_status_e) ov_infer_request_wait(ov_infer_request_t* infer_request);
OPENVINO_C_API(ov_status_e) ov_infer_request_wait_for(ov_infer_request_t* infer_request, const int64_t timeout);
OPENVINO_C_API(ov_status_e) ov_infer_request_set_callback(ov_infer_request_t* infer_request, const ov_callback_t* callback);
OPENVINO_C_API(void) ov_infer_request_free(ov_infer_request_t* infer_request);
OPENVINO_C_API(ov_status_e) ov_infer_request_get_profiling_info(const ov_infer_request_t* infer_request, ov_profiling_info_list_t* profiling_infos);
OPENVINO_C_API(void) ov_profiling_info_list_free(ov_profiling_info_list_t* profiling_infos);
OPENVINO_C_API(ov_status_e) ov_infer_request_reset_state(ov_infer_request_t* infer_request);

/* ---- tensor */
OPENVINO_C_API(ov_status_e) ov_tensor_create_from_host_ptr(const ov_element_type_e type, const ov_shape_t shape, void* host_ptr, ov_tensor_t** tensor);
OPENVINO_C_API(ov_status_e) ov_tensor_create(const ov_element_type_e type, const ov_shape_t shape, ov_tensor_t** tensor);
OPENVINO_C_API(ov_status_e) ov_tensor_set_shape(ov_tensor_t* tensor, const ov_shape_t shape);
OPENVINO_C_API(ov_status_e) ov_tensor_get_shape(const ov_tensor_t* tensor, ov_shape_t* shape);
OPENVINO_C_API(ov_status_e) ov_tensor_get_element_type(const ov_tensor_t* tensor, ov_element_type_e* type);
OPENVINO_C_API(ov_status_e) ov_tensor_get_size(const ov_tensor_t* tensor, size_t* elements_size);
OPENVINO_C_API(ov_status_e) ov_tensor_get_byte_size(const ov_tensor_t* tensor, size_t* byte_size);
OPENVINO_C_API(ov_status_e) ov_tensor_data(const ov_tensor_t* tensor, void** data);
OPENVINO_C_API(void) ov_tensor_free(ov_tensor_t* tensor);

/* ---- pre/post-processing (mean / scale / element type / layout conversion of one input) */
OPENVINO_C_API(ov_status_e) ov_preprocess_prepostprocessor_create(const ov_model_t* model, ov_preprocess_prepostprocessor_t** preprocess);
OPENVINO_C_API(void) ov_preprocess_prepostprocessor_free(ov_preprocess_prepostprocessor_t* preprocess);
OPENVINO_C_API(ov_status_e) ov_preprocess_prepostprocessor_set_input_element_type(ov_preprocess_prepostprocessor_t* preprocess, size_t input, ov_element_type_e type);
OPENVINO_C_API(ov_status_e) ov_preprocess_prepostprocessor_set_input_mean_scale(ov_preprocess_prepostprocessor_t* preprocess, size_t input, const float* mean,
                                                                                const float* scale, size_t channels, int64_t channel_axis);
OPENVINO_C_API(ov_status_e) ov_preprocess_prepostprocessor_set_input_nhwc(ov_preprocess_prepostprocessor_t* preprocess, size_t input);
OPENVINO_C_API(ov_status_e) ov_preprocess_prepostprocessor_build(const ov_preprocess_prepostprocessor_t* preprocess, ov_model_t** model);

#ifdef __cplusplus
}
#endif
#endif
