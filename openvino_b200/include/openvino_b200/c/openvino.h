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
#include <wchar.h>
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
typedef struct ov_preprocess_input_info ov_preprocess_input_info_t;
typedef struct ov_preprocess_input_tensor_info ov_preprocess_input_tensor_info_t;
typedef struct ov_preprocess_preprocess_steps ov_preprocess_preprocess_steps_t;
typedef struct ov_preprocess_input_model_info ov_preprocess_input_model_info_t;
typedef struct ov_preprocess_output_info ov_preprocess_output_info_t;
typedef struct ov_preprocess_output_tensor_info ov_preprocess_output_tensor_info_t;
typedef struct ov_layout ov_layout_t;
typedef struct ov_remote_context ov_remote_context_t;

typedef enum {
    UNDEFINE = 0U, NV12_SINGLE_PLANE, NV12_TWO_PLANES, I420_SINGLE_PLANE, I420_THREE_PLANES, RGB, BGR, GRAY, RGBX, BGRX,
} ov_color_format_e;
typedef enum { RESIZE_LINEAR, RESIZE_CUBIC, RESIZE_NEAREST } ov_preprocess_resize_algorithm_e;
typedef enum { CONSTANT = 0, EDGE, REFLECT, SYMMETRIC } ov_padding_mode_e;

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

/* ---- pre/post-processing, object by object: prepostprocessor -> input info -> tensor info / steps / model info */
OPENVINO_C_API(ov_status_e) ov_preprocess_prepostprocessor_get_input_info(const ov_preprocess_prepostprocessor_t* preprocess, ov_preprocess_input_info_t** info);
OPENVINO_C_API(ov_status_e) ov_preprocess_prepostprocessor_get_input_info_by_name(const ov_preprocess_prepostprocessor_t* preprocess, const char* tensor_name,
                                                                                  ov_preprocess_input_info_t** info);
OPENVINO_C_API(ov_status_e) ov_preprocess_prepostprocessor_get_input_info_by_index(const ov_preprocess_prepostprocessor_t* preprocess, const size_t tensor_index,
                                                                                   ov_preprocess_input_info_t** info);
OPENVINO_C_API(void) ov_preprocess_input_info_free(ov_preprocess_input_info_t* info);
OPENVINO_C_API(ov_status_e) ov_preprocess_input_info_get_tensor_info(const ov_preprocess_input_info_t* info, ov_preprocess_input_tensor_info_t** tensor_info);
OPENVINO_C_API(void) ov_preprocess_input_tensor_info_free(ov_preprocess_input_tensor_info_t* tensor_info);
OPENVINO_C_API(ov_status_e) ov_preprocess_input_info_get_preprocess_steps(const ov_preprocess_input_info_t* info, ov_preprocess_preprocess_steps_t** steps);
OPENVINO_C_API(void) ov_preprocess_preprocess_steps_free(ov_preprocess_preprocess_steps_t* steps);
OPENVINO_C_API(ov_status_e) ov_preprocess_input_info_get_model_info(const ov_preprocess_input_info_t* info, ov_preprocess_input_model_info_t** model_info);
OPENVINO_C_API(void) ov_preprocess_input_model_info_free(ov_preprocess_input_model_info_t* model_info);
OPENVINO_C_API(ov_status_e) ov_preprocess_input_model_info_set_layout(ov_preprocess_input_model_info_t* model_info, ov_layout_t* layout);
OPENVINO_C_API(ov_status_e) ov_preprocess_input_tensor_info_set_element_type(ov_preprocess_input_tensor_info_t* tensor_info, const ov_element_type_e type);
OPENVINO_C_API(ov_status_e) ov_preprocess_input_tensor_info_set_layout(ov_preprocess_input_tensor_info_t* tensor_info, ov_layout_t* layout);
OPENVINO_C_API(ov_status_e) ov_preprocess_input_tensor_info_set_color_format(ov_preprocess_input_tensor_info_t* tensor_info, const ov_color_format_e format);
OPENVINO_C_API(ov_status_e) ov_preprocess_input_tensor_info_set_color_format_with_subname(ov_preprocess_input_tensor_info_t* tensor_info, const ov_color_format_e format,
                                                                                          const size_t sub_names_size, ...);
OPENVINO_C_API(ov_status_e) ov_preprocess_input_tensor_info_set_spatial_static_shape(ov_preprocess_input_tensor_info_t* tensor_info, const size_t height,
                                                                                     const size_t width);
OPENVINO_C_API(ov_status_e) ov_preprocess_input_tensor_info_set_memory_type(ov_preprocess_input_tensor_info_t* tensor_info, const char* mem_type);
OPENVINO_C_API(ov_status_e) ov_preprocess_input_tensor_info_set_from(ov_preprocess_input_tensor_info_t* tensor_info, const ov_tensor_t* tensor);
OPENVINO_C_API(ov_status_e) ov_preprocess_preprocess_steps_resize(ov_preprocess_preprocess_steps_t* steps, const ov_preprocess_resize_algorithm_e algorithm);
OPENVINO_C_API(ov_status_e) ov_preprocess_preprocess_steps_scale(ov_preprocess_preprocess_steps_t* steps, float value);
OPENVINO_C_API(ov_status_e) ov_preprocess_preprocess_steps_scale_multi_channels(ov_preprocess_preprocess_steps_t* steps, const float* values, const int32_t size);
OPENVINO_C_API(ov_status_e) ov_preprocess_preprocess_steps_mean(ov_preprocess_preprocess_steps_t* steps, float value);
OPENVINO_C_API(ov_status_e) ov_preprocess_preprocess_steps_mean_multi_channels(ov_preprocess_preprocess_steps_t* steps, const float* values, const int32_t size);
OPENVINO_C_API(ov_status_e) ov_preprocess_preprocess_steps_crop(ov_preprocess_preprocess_steps_t* steps, int32_t* begin, int32_t begin_size, int32_t* end,
                                                                int32_t end_size);
OPENVINO_C_API(ov_status_e) ov_preprocess_preprocess_steps_convert_layout(ov_preprocess_preprocess_steps_t* steps, ov_layout_t* layout);
OPENVINO_C_API(ov_status_e) ov_preprocess_preprocess_steps_reverse_channels(ov_preprocess_preprocess_steps_t* steps);
OPENVINO_C_API(ov_status_e) ov_preprocess_preprocess_steps_convert_element_type(ov_preprocess_preprocess_steps_t* steps, const ov_element_type_e type);
OPENVINO_C_API(ov_status_e) ov_preprocess_preprocess_steps_convert_color(ov_preprocess_preprocess_steps_t* steps, const ov_color_format_e format);
OPENVINO_C_API(ov_status_e) ov_preprocess_preprocess_steps_pad(const ov_preprocess_preprocess_steps_t* steps, const int* const pads_begin, size_t pads_begin_size,
                                                               const int* const pads_end, size_t pads_end_size, float value, ov_padding_mode_e mode);
OPENVINO_C_API(ov_status_e) ov_preprocess_prepostprocessor_get_output_info(const ov_preprocess_prepostprocessor_t* preprocess, ov_preprocess_output_info_t** info);
OPENVINO_C_API(ov_status_e) ov_preprocess_prepostprocessor_get_output_info_by_index(const ov_preprocess_prepostprocessor_t* preprocess, const size_t tensor_index,
                                                                                    ov_preprocess_output_info_t** info);
OPENVINO_C_API(ov_status_e) ov_preprocess_prepostprocessor_get_output_info_by_name(const ov_preprocess_prepostprocessor_t* preprocess, const char* tensor_name,
                                                                                   ov_preprocess_output_info_t** info);
OPENVINO_C_API(void) ov_preprocess_output_info_free(ov_preprocess_output_info_t* info);
OPENVINO_C_API(ov_status_e) ov_preprocess_output_info_get_tensor_info(const ov_preprocess_output_info_t* info, ov_preprocess_output_tensor_info_t** tensor_info);
OPENVINO_C_API(void) ov_preprocess_output_tensor_info_free(ov_preprocess_output_tensor_info_t* tensor_info);
OPENVINO_C_API(ov_status_e) ov_preprocess_output_set_element_type(ov_preprocess_output_tensor_info_t* tensor_info, const ov_element_type_e type);

/* ---- layouts ("NCHW", "[N,H,W,C]") */
OPENVINO_C_API(ov_status_e) ov_layout_create(const char* layout_desc, ov_layout_t** layout);
OPENVINO_C_API(void) ov_layout_free(ov_layout_t* layout);
OPENVINO_C_API(const char*) ov_layout_to_string(const ov_layout_t* layout);

/* ---- string tensors, ports of either constness, wide-character paths, log callback */
OPENVINO_C_API(ov_status_e) ov_tensor_create_from_string_array(const char** string_array, const size_t array_size, const ov_shape_t shape, ov_tensor_t** tensor);
OPENVINO_C_API(ov_status_e) ov_tensor_set_string_data(ov_tensor_t* tensor, const char** string_array, const size_t array_size);
OPENVINO_C_API(ov_status_e) ov_model_reshape_by_ports(const ov_model_t* model, const ov_output_port_t** output_ports, const ov_partial_shape_t* partial_shapes,
                                                      size_t size);
OPENVINO_C_API(ov_status_e) ov_infer_request_set_tensor_by_port(ov_infer_request_t* infer_request, const ov_output_port_t* port, const ov_tensor_t* tensor);
OPENVINO_C_API(ov_status_e) ov_infer_request_get_tensor_by_port(const ov_infer_request_t* infer_request, const ov_output_port_t* port, ov_tensor_t** tensor);
OPENVINO_C_API(ov_status_e) ov_core_create_with_config_unicode(const wchar_t* xml_config_file, ov_core_t** core);
OPENVINO_C_API(ov_status_e) ov_core_read_model_unicode(const ov_core_t* core, const wchar_t* model_path, const wchar_t* bin_path, ov_model_t** model);
OPENVINO_C_API(ov_status_e) ov_core_compile_model_from_file_unicode(const ov_core_t* core, const wchar_t* model_path, const char* device_name,
                                                                    const size_t property_args_size, ov_compiled_model_t** compiled_model, ...);
OPENVINO_C_API(void) ov_util_set_log_callback(void (*callback)(const char*));
OPENVINO_C_API(void) ov_util_reset_log_callback();

/* ---- device memory contexts and extension libraries: the host device of this library has neither; the calls answer
 *      NOT_IMPLEMENTED with a message (the CUDA device's remote tensors are reached through the Python and C++ APIs) */
OPENVINO_C_API(ov_status_e) ov_core_add_extension(const ov_core_t* core, const char* path);
OPENVINO_C_API(ov_status_e) ov_core_create_context(const ov_core_t* core, const char* device_name, const size_t context_args_size, ov_remote_context_t** context, ...);
OPENVINO_C_API(ov_status_e) ov_core_get_default_context(const ov_core_t* core, const char* device_name, ov_remote_context_t** context);
OPENVINO_C_API(ov_status_e) ov_core_compile_model_with_context(const ov_core_t* core, const ov_model_t* model, const ov_remote_context_t* context,
                                                               const size_t property_args_size, ov_compiled_model_t** compiled_model, ...);
OPENVINO_C_API(ov_status_e) ov_compiled_model_get_context(const ov_compiled_model_t* compiled_model, ov_remote_context_t** context);
OPENVINO_C_API(void) ov_remote_context_free(ov_remote_context_t* context);
OPENVINO_C_API(ov_status_e) ov_remote_context_get_device_name(const ov_remote_context_t* context, char** device_name);
OPENVINO_C_API(ov_status_e) ov_remote_context_get_params(const ov_remote_context_t* context, size_t* size, char** params);
OPENVINO_C_API(ov_status_e) ov_remote_context_create_tensor(const ov_remote_context_t* context, const ov_element_type_e type, const ov_shape_t shape,
                                                            const size_t object_args_size, ov_tensor_t** remote_tensor, ...);
OPENVINO_C_API(ov_status_e) ov_remote_context_create_host_tensor(const ov_remote_context_t* context, const ov_element_type_e type, const ov_shape_t shape,
                                                                 ov_tensor_t** tensor);
OPENVINO_C_API(ov_status_e) ov_remote_tensor_get_params(ov_tensor_t* tensor, size_t* size, char** params);
OPENVINO_C_API(ov_status_e) ov_remote_tensor_get_device_name(ov_tensor_t* remote_tensor, char** device_name);

#ifdef __cplusplus
}
#endif
#endif
