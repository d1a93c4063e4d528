/* Reads an IR model, feeds one tensor, prints the top results.
 *
 *   cc hello_classification.c -I<pkg>/include -L<pkg>/lib -lopenvino_b200_c -o hello_classification
 *   ./hello_classification model.xml [device]
 *
 * The input is filled with a deterministic ramp (there is no image decoder in the C runtime); a real
 * application copies its pixels into ov_tensor_data() instead. Same flow as the reference sample
 * samples/c/hello_classification/main.c: read -> pre-process -> compile -> infer -> top-N.
 */
#include <stdio.h>
#include <stdlib.h>

#include "openvino_b200/c/openvino.h"

#define CHECK(call)                                                                          \
    do {                                                                                     \
        ov_status_e s_ = (call);                                                             \
        if (s_ != OK) {                                                                      \
            const char* m_ = ov_get_last_err_msg();                                          \
            fprintf(stderr, "%s failed: %s (%s)\n", #call, ov_get_error_info(s_), m_);       \
            ov_free(m_);                                                                     \
            return 1;                                                                        \
        }                                                                                    \
    } while (0)

int main(int argc, char** argv) {
    if (argc < 2) {
        fprintf(stderr, "usage: %s model.xml [device]\n", argv[0]);
        return 2;
    }
    const char* device = argc > 2 ? argv[2] : "CPU";
    ov_core_t* core = NULL;
    ov_model_t* model = NULL;
    ov_compiled_model_t* compiled = NULL;
    ov_infer_request_t* request = NULL;
    ov_output_const_port_t* in_port = NULL;
    ov_tensor_t *input = NULL, *output = NULL;
    ov_shape_t in_shape, out_shape;
    ov_element_type_e in_type;

    ov_version_t version;
    CHECK(ov_get_openvino_version(&version));
    printf("runtime: %s\n", version.buildNumber);
    ov_version_free(&version);

    CHECK(ov_core_create(&core));
    CHECK(ov_core_read_model(core, argv[1], NULL, &model));
    CHECK(ov_model_const_input(model, &in_port));
    CHECK(ov_const_port_get_shape(in_port, &in_shape));
    CHECK(ov_port_get_element_type(in_port, &in_type));
    if (in_type != F32) {
        fprintf(stderr, "this sample feeds f32 data\n");
        return 1;
    }
    CHECK(ov_core_compile_model(core, model, device, 0, &compiled));
    CHECK(ov_compiled_model_create_infer_request(compiled, &request));
    CHECK(ov_tensor_create(F32, in_shape, &input));
    {
        float* data = NULL;
        size_t n = 0, i;
        CHECK(ov_tensor_data(input, (void**)&data));
        CHECK(ov_tensor_get_size(input, &n));
        for (i = 0; i < n; ++i) data[i] = (float)(i % 255) / 255.0f;
    }
    CHECK(ov_infer_request_set_input_tensor_by_index(request, 0, input));
    CHECK(ov_infer_request_infer(request));
    CHECK(ov_infer_request_get_output_tensor_by_index(request, 0, &output));
    CHECK(ov_tensor_get_shape(output, &out_shape));
    {
        const float* scores = NULL;
        size_t n = 0, i, k;
        CHECK(ov_tensor_data(output, (void**)&scores));
        CHECK(ov_tensor_get_size(output, &n));
        printf("top results (of %zu):\n", n);
        {
            size_t picked[3] = {(size_t)-1, (size_t)-1, (size_t)-1};
            for (k = 0; k < 3 && k < n; ++k) {
                size_t best = (size_t)-1;
                for (i = 0; i < n; ++i) {
                    if (i == picked[0] || i == picked[1] || i == picked[2]) continue;
                    if (best == (size_t)-1 || scores[i] > scores[best]) best = i;
                }
                picked[k] = best;
                printf("  class %zu: %.6f\n", best, scores[best]);
            }
        }
    }
    ov_shape_free(&in_shape);
    ov_shape_free(&out_shape);
    ov_tensor_free(input);
    ov_tensor_free(output);
    ov_output_const_port_free(in_port);
    ov_infer_request_free(request);
    ov_compiled_model_free(compiled);
    ov_model_free(model);
    ov_core_free(core);
    return 0;
}
