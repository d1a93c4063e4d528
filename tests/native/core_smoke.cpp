// Native smoke test of the core library for sanitizer builds (no Python in the process): read a model through the C API,
// query it, reshape, compile on the host device, run synchronous and asynchronous inference from several threads, save
// and re-read it; then drive the continuous-batching scheduler (preemption, prefix cache) through a few hundred steps.
// Built by tests/test_sanitizers.py with -fsanitize=address,undefined and with -fsanitize=thread.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "openvino_b200/c/openvino.h"
#include "sched.hpp"

#define CHECK(expr)                                                                              \
    do {                                                                                         \
        ov_status_e _s = (expr);                                                                 \
        if (_s != 0) {                                                                           \
            std::fprintf(stderr, "%s failed (%d): %s\n", #expr, (int)_s, ov_get_last_err_msg()); \
            std::exit(2);                                                                        \
        }                                                                                        \
    } while (0)

static void infer_worker(ov_compiled_model_t* cm, int iters, float fill, std::vector<float>* first_out) {
    ov_infer_request_t* req = nullptr;
    CHECK(ov_compiled_model_create_infer_request(cm, &req));
    ov_tensor_t* in = nullptr;
    CHECK(ov_infer_request_get_input_tensor(req, &in));
    void* data = nullptr;
    size_t bytes = 0;
    CHECK(ov_tensor_data(in, &data));
    CHECK(ov_tensor_get_byte_size(in, &bytes));
    float* f = static_cast<float*>(data);
    for (size_t i = 0; i < bytes / sizeof(float); ++i) f[i] = fill + 0.001f * (float)(i % 97);
    for (int it = 0; it < iters; ++it) {
        if (it % 2 == 0) {
            CHECK(ov_infer_request_infer(req));
        } else {
            CHECK(ov_infer_request_start_async(req));
            CHECK(ov_infer_request_wait(req));
        }
        ov_tensor_t* out = nullptr;
        CHECK(ov_infer_request_get_output_tensor(req, &out));
        void* od = nullptr;
        size_t ob = 0;
        CHECK(ov_tensor_data(out, &od));
        CHECK(ov_tensor_get_byte_size(out, &ob));
        const float* of = static_cast<const float*>(od);
        if (it == 0) first_out->assign(of, of + ob / sizeof(float));
        else
            for (size_t i = 0; i < ob / sizeof(float); ++i)
                if (of[i] != (*first_out)[i]) { std::fprintf(stderr, "output changed between iterations\n"); std::exit(3); }
        ov_tensor_free(out);
    }
    ov_tensor_free(in);
    ov_infer_request_free(req);
}

static void scheduler_run(bool split_fuse, bool prefix) {
    ovc::SchedulerConfig cfg;
    cfg.max_num_batched_tokens = 24;
    cfg.max_num_seqs = 4;
    cfg.num_kv_blocks = 9;
    cfg.block_size = 4;
    cfg.dynamic_split_fuse = split_fuse;
    cfg.enable_prefix_caching = prefix;
    ovc::Scheduler s(cfg);
    std::vector<ovc::SeqPtr> seqs;
    for (int r = 0; r < 9; ++r) {
        std::vector<int32_t> prompt;
        for (int i = 0; i < 6 + (r * 5) % 9; ++i) prompt.push_back(i < 8 ? 100 + i : 7 * r + i);   // a common 8-token prefix
        seqs.push_back(s.add(r, prompt, 5, /*eos=*/3, /*ignore_eos=*/r % 2 == 0));
    }
    ovc::DescLayout lay;
    int64_t off = 0;
    auto field = [&](int64_t& f, int64_t n) { f = off; off += (n + 3) / 4 * 4; };
    lay.Tcap = 24; lay.Bcap = 4; lay.blocks_cap = 4 * 8;
    field(lay.ids, 24); field(lay.positions, 24); field(lay.slot_map, 24); field(lay.tok_src, 24); field(lay.tok_dst, 4);
    field(lay.logit_idx, 4); field(lay.past_lens, 4); field(lay.subsequence_begins, 5); field(lay.block_indices_begins, 5);
    field(lay.block_indices, 32);
    std::vector<int32_t> desc((size_t)off);
    int steps = 0;
    while (s.has_unfinished()) {
        ovc::ScheduledStep st;
        if (!s.schedule(st)) { std::fprintf(stderr, "scheduler stalled\n"); std::exit(4); }
        s.fill(st, desc.data(), lay, false);
        std::vector<int32_t> toks(st.seqs.size());
        for (size_t i = 0; i < toks.size(); ++i) toks[i] = (int32_t)((steps + (int)i) % 6);   // 3 = end of sequence now and then
        auto produced = s.commit(st, nullptr);
        s.patch(produced, toks.data());
        if (++steps > 2000) { std::fprintf(stderr, "scheduler does not terminate\n"); std::exit(4); }
    }
    if (s.num_free_blocks() != cfg.num_kv_blocks) { std::fprintf(stderr, "blocks leaked: %lld free\n", (long long)s.num_free_blocks()); std::exit(4); }
    for (auto& q : seqs) if (!q->finished) { std::fprintf(stderr, "sequence not finished\n"); std::exit(4); }
}

int main(int argc, char** argv) {
    if (argc < 3) { std::fprintf(stderr, "usage: %s model.xml out.xml\n", argv[0]); return 1; }
    ov_core_t* core = nullptr;
    CHECK(ov_core_create(&core));
    ov_model_t* model = nullptr;
    CHECK(ov_core_read_model(core, argv[1], nullptr, &model));
    size_t n_in = 0, n_out = 0;
    CHECK(ov_model_inputs_size(model, &n_in));
    CHECK(ov_model_outputs_size(model, &n_out));
    if (n_in != 1 || n_out != 1) { std::fprintf(stderr, "expected one input and one output\n"); return 2; }
    ov_output_const_port_t* port = nullptr;
    CHECK(ov_model_const_input(model, &port));
    char* name = nullptr;
    CHECK(ov_port_get_any_name(port, &name));
    ov_free(name);
    ov_output_const_port_free(port);
    // reshape the batch, compile, run from four threads at once
    const int64_t dims[4] = {2, 3, 8, 8};
    ov_partial_shape_t ps;
    CHECK(ov_partial_shape_create_static(4, dims, &ps));
    CHECK(ov_model_reshape_single_input(model, ps));
    ov_partial_shape_free(&ps);
    ov_compiled_model_t* cm = nullptr;
    CHECK(ov_core_compile_model(core, model, "CPU", 0, &cm));
    std::vector<std::vector<float>> outs(4);
    std::vector<std::thread> th;
    for (int t = 0; t < 4; ++t) th.emplace_back(infer_worker, cm, 6, 0.25f * (float)(t % 2), &outs[t]);
    for (auto& t : th) t.join();
    if (outs[0] != outs[2] || outs[1] != outs[3] || outs[0] == outs[1]) { std::fprintf(stderr, "threads disagree\n"); return 3; }
    CHECK(ov_model_save(model, argv[2], false));
    ov_model_t* again = nullptr;
    CHECK(ov_core_read_model(core, argv[2], nullptr, &again));
    ov_model_free(again);
    ov_compiled_model_free(cm);
    ov_model_free(model);
    ov_core_free(core);
    for (int sf = 0; sf < 2; ++sf)
        for (int pc = 0; pc < 2; ++pc) scheduler_run(sf != 0, pc != 0);
    std::printf("CORE_SMOKE_OK\n");
    return 0;
}
